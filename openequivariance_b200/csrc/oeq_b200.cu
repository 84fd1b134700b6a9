// Host side of the oeq_b200 C ABI (declared in include/oeq_b200.h):
//   descriptor parser -> problem header emitter -> NVRTC (sm_100a) -> cubin cache -> launches.
//
// The device code lives in kernels/*.cuh (hand-written templates).  The only generated text is the short
// "problem header": constexpr tables for the irreps / instructions and one straight-line function per
// instruction holding its sparse Clebsch-Gordan contraction with the coefficients as literals.
//
// Counterparts in the reference: extension/backend/backend_cuda.hpp:154-361 (CUJITKernel: NVRTC, module
// load, launch), extension/tensorproducts.hpp:10-113 and extension/convolution.hpp:15-179 (kernel lists and
// launch sequences), extension/torch_core.hpp:180-270 (hash-keyed caches under a mutex).

#include <cuda_runtime.h>
#include <nvrtc.h>
#include <dlfcn.h>
#include <sys/stat.h>
#include <unistd.h>

#include <algorithm>
#include <atomic>
#include <cstdarg>
#include <cstdint>
#include <cstdio>
#include <cstdlib>
#include <cstring>
#include <map>
#include <memory>
#include <mutex>
#include <set>
#include <tuple>
#include <sstream>
#include <string>
#include <vector>

#include "../../include/oeq_b200.h"
#include "kernels_embed.inc"  // generated at build time: K_COMMON, K_GENERIC, K_FAST_UVU as raw strings
#include "graph_prep.cuh"         // problem-independent kernels: grouping / sorting of edge lists
#include "partition_plan.cuh"     // ... and the plans of the partitioned / streamed drivers
#include "group_mm.cuh"       // problem-independent kernels: ragged grouped products of the symmetric contraction

namespace {

// ------------------------------------------------------------------------------------------------ errors
thread_local std::string g_err;
std::atomic<long long> g_launches{0};
bool g_log = false;
bool g_force_generic = false;
bool g_no_tc = false;          // tuning aid: keep 'uvw' forward on the general kernel
int g_tc_backward = 7;         // 'uvw' backward outputs taken from the tensor-core kernels: 1 dx, 2 dy, 4 dW (bit mask)
bool g_single_group = false;   // tuning aid: one thread group per edge on the channel-parallel path
bool g_single_producer = false;   // tuning aid: one producer warp per CTA in the forward kernels too
int g_validate = 1;            // index checks of convolution calls: 0 never, 1 first call per edge list, 2 every call
bool g_streams_fwd = false;    // the forward kernels take part in `streams` too (the backward kernels always do)
int g_streams = 1;             // edge streams per CTA on the channel-parallel path (1: two CTAs per SM; 2-4: one CTA with
                               // that many consumer sets and a register hand-over; measured slower on the benchmark graph)
std::string g_cache_dir;
std::mutex g_mutex;

int fail(int code, const char* fmt, ...) {
    char buf[4096];
    va_list ap;
    va_start(ap, fmt);
    vsnprintf(buf, sizeof buf, fmt, ap);
    va_end(ap);
    g_err = buf;
    if (g_log) fprintf(stderr, "[oeq_b200] error %d: %s\n", code, buf);
    return code;
}

#define CUDA_TRY(expr)                                                                              \
    do {                                                                                            \
        cudaError_t _e = (expr);                                                                    \
        if (_e != cudaSuccess) return fail(OEQB_ECUDA, "%s failed: %s", #expr, cudaGetErrorString(_e)); \
    } while (0)

// -------------------------------------------------------------------------------------------- descriptor
struct Block { int mul, l, p, off; int d() const { return 2 * l + 1; } };
struct Nz { int i, j, k; double c; };
struct Instr { int a, b, o; long long woff; std::vector<Nz> nz; };
// Distinct (i, k) index pairs of an instruction's Clebsch-Gordan nonzeros, sorted, each with the nonzeros (one per j)
// that share it.  The channel-parallel kernels fold the edge's y into one coefficient per pair.
struct IkPair { int i, k; std::vector<Nz> terms; };
std::vector<IkPair> ik_pairs(const Instr& I) {
    std::vector<Nz> v = I.nz;
    std::stable_sort(v.begin(), v.end(), [](const Nz& a, const Nz& b) { return a.i != b.i ? a.i < b.i : a.k < b.k; });
    std::vector<IkPair> out;
    for (const Nz& q : v) {
        if (out.empty() || out.back().i != q.i || out.back().k != q.k) out.push_back(IkPair{q.i, q.k, {}});
        out.back().terms.push_back(q);
    }
    return out;
}
struct Desc {
    int dtype = 1, layout = 0, shared = 0, uvw = 0, conv = 0, det = 0, kahan = 0, idx = 4;
    std::vector<Block> L[3];
    long long dim[3] = {0, 0, 0};
    long long wn = 0;
    std::vector<Instr> ins;
    bool fast = false;   // channel-parallel pipelined kernels applicable
    int fast_U = 0;      // common multiplicity on the fast path
    int fast_S = 0;      // shared-memory stages per CTA
    int fast_ctas = 0;   // resident CTAs per SM the stages are sized for
    int fast_ncy = 0;    // folded-coefficient slots per edge (each instruction padded to a multiple of 4)
    int fast_ng = 1;     // thread groups sharing an edge
    int fast_ch = 1;     // channels carried by one consumer thread
    int fast_bwd_ng = 1; // thread groups of the backward kernels (2 in the fp64 configuration)
    int fastb_S = 0, fastb_ctas = 0;   // stages / resident CTAs of the first-order backward kernels (differ from the forward's
    size_t fastb_smem = 0;            // only for compensated summation, whose forward alone needs the wide configuration)
    size_t fast_smem = 0;
    bool tc = false;         // tensor-core 'uvw' forward applicable (shared weights, 32-wide multiplicities, fp32)
    bool tc_bwd = false;     // ... and the tensor-core backward kernels
    bool tc_zero_z = false, tc_zero_dx = false;   // some output / input block has no path: zero the result first
    int tc_ngrp = 0;         // groups of the tensor-core weight-gradient kernel (16 per launch)
    size_t tc_smem[3] = {0, 0, 0}, tc_dw_smem = 0;   // dynamic shared memory of the tensor-core programs
    int fast_S3 = 0;         // stages of the atomic forward kernel (it also holds one output row for the bulk reduce)
    size_t fast_smem3 = 0;
    int fast_S4 = 0;         // stages of the second-order kernels (their stage carries a second coefficient table)
    size_t fast_smem4 = 0;
    int fast_V = 1;          // edge streams per CTA of the first-order kernels (see kernels/fast_uvu.cuh); 1 = none
    int fast_SV = 0;         // stages per stream when fast_V > 1
    size_t fast_smemV = 0;
    size_t elt() const { return dtype == 2 ? 8 : 4; }
};

std::vector<std::vector<int>> tc_dw_groups(const Desc& d, size_t* xs_floats);
size_t tc_smem_bytes(const Desc& d, int mode);
size_t tc_dw_smem_bytes(const Desc& d);
size_t tc_smem_base_bytes(const Desc& d, int mode);
int tc_xs2_d1(const Desc& d, int mode, size_t base);

bool parse_desc(const char* text, size_t len, Desc& d, std::string& why) {
    std::istringstream in(std::string(text, len));
    std::string tok;
    auto bad = [&](const char* m) { why = m; return false; };
    int version = 0;
    if (!(in >> tok >> version) || tok != "OEQB" || version != 1) return bad("missing 'OEQB 1' header");
    std::string mode;
    if (!(in >> tok >> d.dtype) || tok != "dtype" || (d.dtype != 1 && d.dtype != 2)) return bad("bad dtype");
    if (!(in >> tok >> d.layout) || tok != "layout") return bad("bad layout");
    if (!(in >> tok >> d.shared) || tok != "shared") return bad("bad shared");
    if (!(in >> tok >> mode) || tok != "mode" || (mode != "uvu" && mode != "uvw")) return bad("bad mode");
    d.uvw = mode == "uvw";
    if (!(in >> tok >> d.conv >> d.det >> d.kahan >> d.idx) || tok != "conv" || (d.idx != 3 && d.idx != 4))
        return bad("bad conv line");
    const char* tags[3] = {"L1", "L2", "L3"};
    for (int r = 0; r < 3; ++r) {
        int n = 0;
        if (!(in >> tok >> n >> d.dim[r]) || tok != tags[r] || n < 0 || n > 4096) return bad("bad irreps header");
        long long off = 0;
        for (int b = 0; b < n; ++b) {
            Block blk{};
            if (!(in >> blk.mul >> blk.l >> blk.p >> blk.off) || blk.mul < 0 || blk.l < 0 || blk.l > 32)
                return bad("bad irreps block");
            if (blk.off != off) return bad("irreps offsets are not contiguous");
            off += (long long)blk.mul * blk.d();
            d.L[r].push_back(blk);
        }
        if (off != d.dim[r]) return bad("irreps dim mismatch");
    }
    if (!(in >> tok >> d.wn) || tok != "wn" || d.wn < 0) return bad("bad wn");
    int nins = 0;
    if (!(in >> tok >> nins) || tok != "ins" || nins <= 0 || nins > 65536) return bad("bad ins count");
    long long wsum = 0;
    for (int n = 0; n < nins; ++n) {
        Instr I{};
        int nnz = 0;
        if (!(in >> tok >> I.a >> I.b >> I.o >> I.woff >> nnz) || tok != "I") return bad("bad instruction line");
        if (I.a < 0 || I.a >= (int)d.L[0].size() || I.b < 0 || I.b >= (int)d.L[1].size() || I.o < 0 ||
            I.o >= (int)d.L[2].size() || nnz < 0)
            return bad("instruction index out of range");
        const Block &A = d.L[0][I.a], &B = d.L[1][I.b], &O = d.L[2][I.o];
        if (!d.uvw && A.mul != O.mul) return bad("uvu needs mul(in1) == mul(out)");
        if (I.woff != wsum) return bad("weight offsets are not contiguous");
        wsum += (long long)A.mul * B.mul * (d.uvw ? O.mul : 1);
        for (int z = 0; z < nnz; ++z) {
            Nz q{};
            std::string hex;
            if (!(in >> q.i >> q.j >> q.k >> hex)) return bad("bad CG entry");
            if (q.i < 0 || q.i >= A.d() || q.j < 0 || q.j >= B.d() || q.k < 0 || q.k >= O.d()) return bad("CG index out of range");
            q.c = strtod(hex.c_str(), nullptr);
            I.nz.push_back(q);
        }
        d.ins.push_back(std::move(I));
    }
    if (wsum != d.wn) return bad("weight_numel mismatch");
    if (!(in >> tok) || tok != "end") return bad("missing 'end'");
    if (d.layout == 1 && d.uvw) return bad("ir_mul layout with uvw");
    if (d.dim[0] * 1LL > (1LL << 24) || d.dim[2] > (1LL << 24) || d.wn > (1LL << 30)) return bad("problem too large");

    // Fast path: fp32 or fp64, either layout, uvu, per-item weights, every in2 multiplicity 1, one common in1 multiplicity
    // that is a multiple of 32, l <= 4 everywhere, rows small enough to live in registers; Kahan summation for the
    // deterministic convolution only (the only place the reference offers it).
    // fp64 takes the "wide" configuration: one channel per thread in two block-owning thread groups (forward and
    // backward), so that half a gradient row of doubles fits a thread's registers, and one CTA per SM for the doubled stages.
    d.fast = false;
    if ((d.dtype == 1 || d.dtype == 2) && !d.uvw && !d.shared && (!d.kahan || (d.conv && d.det && d.dtype == 1)) && !d.L[0].empty()) {
        // compensated summation also takes the wide configuration: sum and compensation of half a row per thread
        const bool wide = d.dtype == 2 || d.kahan;
        bool ok = true;
        int U = d.L[0][0].mul;
        for (auto& b : d.L[0]) ok = ok && b.mul == U && b.l <= 4;
        for (auto& b : d.L[1]) ok = ok && b.mul == 1 && b.l <= 4;
        for (auto& b : d.L[2]) ok = ok && b.mul == U && b.l <= 4;
        ok = ok && U >= 32 && U % 32 == 0 && U <= (wide ? 128 : 256) && d.dim[1] <= 32;
        ok = ok && d.dim[0] / U <= 32 && d.dim[2] / U <= 112;
        if (ok) {
            const size_t elt = d.elt();
            int ncy = 0;
            for (auto& I : d.ins) ncy += ((int)ik_pairs(I).size() + 3) & ~3;
            const int nyp = d.dim[1] <= 1 ? 1 : d.dim[1] <= 2 ? 2 : d.dim[1] <= 4 ? 4 : d.dim[1] <= 8 ? 8 : d.dim[1] <= 16 ? 16 : 32;
            // Two channels per thread halve the shared-memory traffic of the coefficient loads; the row registers
            // that doubles are won back by dealing the blocks to two thread groups.
            const int ch = (!wide && !g_single_group && U % 64 == 0 && d.ins.size() >= 2) ? 2 : 1;
            const int ng = (ch == 2 || (wide && d.ins.size() >= 2 && d.L[0].size() >= 2 && d.L[2].size() >= 2)) ? 2 : 1;
            const int bwd_ng = wide ? ng : 1;
            const int nthreads = std::max(ng * U / ch, bwd_ng * U);
            const size_t stage = ((elt * (size_t)(d.dim[0] + d.wn + ncy + ((d.dim[1] + 3) & ~3) + 8 + (nthreads / 32) * nyp) + 40) + 15) & ~(size_t)15;
            int ctas = wide ? 1 : 256 / U;
            ctas = ctas < 1 ? 1 : (ctas > 4 ? 4 : ctas);
            while (ctas > 1 && ctas * (nthreads + 32) * (ch == 2 ? 168 : 128) > 65536) --ctas;   // registers per thread
            int S = 0;
            for (; ctas >= 1; ctas /= 2) {
                const size_t budget = 232448 / ctas - 1024 - 256;
                S = (int)(budget / (stage + 32));
                if (S > 6) S = 6;
                if (S >= 3) break;
            }
            if (S >= 3 && ctas >= 1 && nthreads + 64 <= 1024) {
                d.fast = true;
                d.fast_U = U; d.fast_S = S; d.fast_ctas = ctas; d.fast_ncy = ncy; d.fast_ng = ng; d.fast_ch = ch;
                d.fast_bwd_ng = bwd_ng;
                d.fast_smem = (size_t)S * (stage + 32) + 160;
                d.fastb_S = S; d.fastb_ctas = ctas; d.fastb_smem = d.fast_smem;
                if (d.kahan && d.dtype == 1) {
                    // Only the forward accumulates over edges; the backward kernel of the compensated variant is the plain one
                    // (one channel per thread, one group) in its own, denser configuration.
                    const int nthreads_b = U;
                    const size_t stage_b = ((elt * (size_t)(d.dim[0] + d.wn + ncy + ((d.dim[1] + 3) & ~3) + 8 + (nthreads_b / 32) * nyp) + 40) + 15) & ~(size_t)15;
                    int ctas_b = 256 / U;
                    ctas_b = ctas_b < 1 ? 1 : (ctas_b > 4 ? 4 : ctas_b);
                    while (ctas_b > 1 && ctas_b * (nthreads_b + 64) * 168 > 65536) --ctas_b;
                    int S_b = 0;
                    for (; ctas_b >= 1; ctas_b /= 2) {
                        S_b = (int)((232448 / ctas_b - 1024 - 256) / (stage_b + 32));
                        if (S_b > 6) S_b = 6;
                        if (S_b >= 3) break;
                    }
                    if (S_b >= 3 && ctas_b >= 1) {
                        d.fast_bwd_ng = 1; d.fastb_S = S_b; d.fastb_ctas = ctas_b; d.fastb_smem = (size_t)S_b * (stage_b + 32) + 160;
                    }
                }
                const size_t stage4 = stage + elt * (size_t)(ncy + ((d.dim[1] + 3) & ~3));
                int S4 = wide ? 0 : (int)((232448 / ctas - 1024 - 256) / (stage4 + 32));
                if (S4 > 6) S4 = 6;
                d.fast_S4 = S4;    // < 3: second-order passes run on the general kernels
                d.fast_smem4 = (size_t)S4 * (stage4 + 32) + 160;
                // Several edge streams in one CTA per SM: consumer sets of exactly one warpgroup, three stages each
                if (!wide && g_streams > 1 && g_streams <= 4 && nthreads == 128 && U == 128) {
                    const int V = g_streams;
                    int cyt = 1;
                    for (auto& I : d.ins)
                        for (auto& pr : ik_pairs(I)) cyt = std::max(cyt, (int)pr.terms.size());
                    const size_t table = (size_t)ncy * cyt * 8;   // consumer-side folding: (coefficient, index) pairs
                    int SV = (int)((((232448 - 1024 - table) / V) - 256) / (stage + 32));
                    if (SV > 4) SV = 4;
                    if (SV >= 3) { d.fast_V = V; d.fast_SV = SV; d.fast_smemV = (size_t)V * ((size_t)SV * (stage + 32) + 128 + 64) + table + 64; }
                }
                int S3 = wide ? 0 : (int)((232448 / ctas - 1024 - 256 - elt * (size_t)d.dim[2]) / (stage + 32));
                if (S3 > 6) S3 = 6;
                d.fast_S3 = S3;    // < 2: atomic forward falls back to the general kernel
                d.fast_smem3 = (size_t)(S3 > 0 ? S3 : 0) * (stage + 32) + elt * (size_t)d.dim[2] + 192;
            }
        }
    }
    // Tensor-core path for 'uvw': shared fp32 weights, every in1 / out multiplicity a multiple of 32 (up to 128: the weight
    // blocks are walked in 32 x 32 tiles), in2 multiplicity 1, l <= 3.
    d.tc = false;
    d.tc_bwd = false;
    if (d.dtype == 1 && d.layout == 0 && d.uvw && d.shared && !d.L[0].empty()) {
        bool ok = d.dim[1] <= 16;
        for (auto& b : d.L[0]) ok = ok && b.mul % 32 == 0 && b.mul <= 128 && b.l <= 3;
        for (auto& b : d.L[1]) ok = ok && b.mul == 1 && b.l <= 3;
        for (auto& b : d.L[2]) ok = ok && b.mul % 32 == 0 && b.mul <= 128 && b.l <= 3;
        // the kernels store only the blocks they accumulate: an output block without a path (or, for the gradient, an input
        // block that no path reads) is zeroed by the host first
        std::vector<int> hit(d.L[2].size(), 0), read(d.L[0].size(), 0);
        for (auto& I : d.ins) { hit[I.o] = 1; read[I.a] = 1; }
        d.tc_zero_z = d.tc_zero_dx = false;
        for (int h : hit) d.tc_zero_z = d.tc_zero_z || !h;
        for (int h : read) d.tc_zero_dx = d.tc_zero_dx || !h;
        long long npath = 0;   // 32 x 32 weight tiles: the per-path tables live in constant memory
        if (ok) for (auto& I : d.ins) npath += (long long)(d.L[0][I.a].mul / 32) * (d.L[2][I.o].mul / 32);
        ok = ok && npath <= 1024 && !d.ins.empty();
        // The tensor cores add into their accumulators with truncation: measured ~1e-6 + 5.5e-9 per accumulated product.  The
        // sums of the forward (per output channel: the channels of every path into its block) and of the gradient of x (per
        // input channel) are kept below 1,280 products, which stays inside the 1e-5 bound.
        if (ok) {
            std::vector<long long> into(d.L[2].size(), 0), from(d.L[0].size(), 0);
            for (auto& I : d.ins) { into[I.o] += d.L[0][I.a].mul; from[I.a] += d.L[2][I.o].mul; }
            for (long long v : into) ok = ok && v <= 1280;
            for (long long v : from) ok = ok && v <= 1280;
        }
        d.tc = ok;
        d.tc_bwd = ok;
        for (int m = 0; m < 3; ++m) d.tc_smem[m] = ok ? tc_smem_bytes(d, m) : 0;
        d.tc = d.tc && d.tc_smem[0] <= 232448;
        d.tc_bwd = d.tc_bwd && d.tc && d.tc_smem[1] <= 232448 && d.tc_smem[2] <= 232448;
        if (d.tc_bwd) { d.tc_ngrp = (int)tc_dw_groups(d, nullptr).size(); d.tc_dw_smem = tc_dw_smem_bytes(d); }
    }
    return true;
}

// ------------------------------------------------------------------------------------------ header emit
std::string hexf(double v) {
    char b[64];
    snprintf(b, sizeof b, "%a", v);
    return b;
}

// Straight-line contraction  out[oidx] += c * (p[pidx] * q[qidx])  grouped so each product is formed once.
void emit_contraction(std::ostringstream& s, const char* name, const char* pn, const char* qn, const char* on,
                      const std::vector<Nz>& nz, int which /*0 fwd, 1 dx, 2 dy*/) {
    s << "  template <class R> static OEQ_DEV void " << name << "(const R* " << pn << ", const R* " << qn << ", R* "
      << on << ") {\n";
    struct E { int p, q, o; double c; };
    std::vector<E> es;
    for (auto& z : nz) {
        if (which == 0) es.push_back({z.i, z.j, z.k, z.c});        // t[k] += c x[i] y[j]
        else if (which == 1) es.push_back({z.j, z.k, z.i, z.c});   // dx[i] += c y[j] g[k]
        else es.push_back({z.i, z.k, z.j, z.c});                   // dy[j] += c x[i] g[k]
    }
    std::stable_sort(es.begin(), es.end(), [](const E& a, const E& b) { return a.p != b.p ? a.p < b.p : a.q < b.q; });
    for (size_t n = 0; n < es.size();) {
        size_t m = n;
        s << "    { const R pr = " << pn << "[" << es[n].p << "] * " << qn << "[" << es[n].q << "];";
        while (m < es.size() && es[m].p == es[n].p && es[m].q == es[n].q) {
            s << " " << on << "[" << es[m].o << "] += R(" << hexf(es[m].c) << ") * pr;";
            ++m;
        }
        s << " }\n";
        n = m;
    }
    s << "  }\n";
}

std::string emit_header(const Desc& d) {
    std::ostringstream s;
    s << "// problem header (generated from the descriptor)\n";
    s << "typedef " << (d.dtype == 2 ? "double" : "float") << " T;\n";
    s << "typedef " << (d.idx == 3 ? "int" : "long long") << " IDX;\n";
    s << "#define OEQ_SHARED_W " << d.shared << "\n#define OEQ_UVW " << d.uvw << "\n#define OEQ_IR_MUL " << d.layout
      << "\n#define OEQ_KAHAN " << d.kahan << "\n";
    s << "#define OEQ_DEV __device__ __forceinline__\n";
    s << "constexpr int L1_DIM = " << d.dim[0] << ", L2_DIM = " << d.dim[1] << ", L3_DIM = " << d.dim[2]
      << ", WN = " << d.wn << ", NINS = " << d.ins.size() << ", NB1 = " << d.L[0].size() << ", NB2 = " << d.L[1].size()
      << ", NB3 = " << d.L[2].size() << ";\n";
    for (int r = 0; r < 3; ++r) {
        s << "template <int B> struct Blk" << (r + 1) << ";\n";
        for (size_t b = 0; b < d.L[r].size(); ++b) {
            const Block& k = d.L[r][b];
            s << "template <> struct Blk" << (r + 1) << "<" << b << "> { static constexpr int MUL = " << k.mul
              << ", D = " << k.d() << ", OFF = " << k.off << "; };\n";
        }
    }
    s << "template <int I> struct Ins;\n";
    for (size_t n = 0; n < d.ins.size(); ++n) {
        const Instr& I = d.ins[n];
        const Block &A = d.L[0][I.a], &B = d.L[1][I.b], &O = d.L[2][I.o];
        s << "template <> struct Ins<" << n << "> {\n";
        s << "  static constexpr int A = " << I.a << ", B = " << I.b << ", O = " << I.o << ", WOFF = " << I.woff
          << ", U = " << A.mul << ", V = " << B.mul << ", WN_ = " << O.mul << ", D1 = " << A.d() << ", D2 = " << B.d()
          << ", D3 = " << O.d() << ", NNZ = " << I.nz.size() << ";\n";
        emit_contraction(s, "fwd", "x", "y", "t", I.nz, 0);
        emit_contraction(s, "dx", "y", "g", "dx", I.nz, 1);
        emit_contraction(s, "dy", "x", "g", "dy", I.nz, 2);
        s << "};\n";
    }
    return s.str();
}

// Tables and per-instruction register kernels for the channel-parallel family (kernels/fast_uvu.cuh).
// cy[i,k] = sum_j C[i,j,k] y[j] is formed once per edge by the producer warp; the consumer code below reads it as float4.
// Producer warps of a kernel with `stages` stages: two from four stages on (its look-ahead is then a multiple of two).
int fast_producers(int stages) { return (stages >= 4 && !g_single_producer) ? 2 : 1; }

std::string emit_fast(const Desc& d, int ch, int ng, bool dbl, int stages, size_t smem_bytes, int streams, int ctas) {
    std::ostringstream s;
    if (!d.fast) { s << "#define OEQ_FAST 0\n"; return s.str(); }
    s << "#define OEQ_FAST 1\n";
    // element type T comes from the problem header; T4 = four of them (16 or 32 bytes), oeq_fma = fused multiply-add on T
    s << "template <class R> struct OeqVec4;\ntemplate <> struct OeqVec4<float> { typedef float4 type; };\n"
         "template <> struct OeqVec4<double> { typedef double4 type; };\ntypedef OeqVec4<T>::type T4;\n"
         "OEQ_DEV T oeq_fma(T a, T b, T c) { return fma(a, b, c); }\n";
    s << "#define FAST_DBL " << (dbl ? 1 : 0) << "\n";
    s << "constexpr int FAST_V = " << streams << ";\n";
    s << "constexpr int FAST_NP = " << (streams > 1 ? 1 : fast_producers(stages)) << ";\n";
    s << "constexpr size_t FAST_SMEM_BYTES = " << smem_bytes << ";\n";
    s << "constexpr int FU = " << d.fast_U << ", NCY = " << d.fast_ncy << ", FAST_S = " << stages
      << ", FAST_CTAS = " << (streams > 1 ? 1 : ctas) << ", FAST_CH = " << ch << ", FAST_XPC = " << d.dim[0] / d.fast_U
      << ", FAST_GPC = " << d.dim[2] / d.fast_U << ";\n";
    // Folded-coefficient table: slot q of an edge holds sum_t FAST_CYC[q][t] * y[FAST_CYJ[q][t]], one slot per (i, k) pair
    std::ostringstream cyc, cyj;
    std::vector<int> cyoff;
    std::vector<std::vector<IkPair>> pairs;
    int off = 0, cyt = 1;
    for (auto& I : d.ins) {
        pairs.push_back(ik_pairs(I));
        for (auto& pr : pairs.back()) cyt = std::max(cyt, (int)pr.terms.size());
    }
    for (size_t n = 0; n < d.ins.size(); ++n) {
        cyoff.push_back(off);
        const int np = (int)pairs[n].size(), pad = (np + 3) & ~3;
        for (int q = 0; q < pad; ++q)
            for (int t = 0; t < cyt; ++t) {
                const bool real = q < np && t < (int)pairs[n][q].terms.size();
                cyc << "T(" << (real ? hexf(pairs[n][q].terms[t].c) : std::string("0.0")) << "), ";
                cyj << (real ? d.L[1][d.ins[n].b].off + pairs[n][q].terms[t].j : 0) << ", ";
            }
        off += pad;
    }
    s << "constexpr int FAST_CYT = " << cyt << ";\n";
    s << "__device__ const T FAST_CYC[NCY * FAST_CYT] = {" << cyc.str() << "};\n";
    s << "__device__ const int FAST_CYJ[NCY * FAST_CYT] = {" << cyj.str() << "};\n";
    s << "template <int I> struct FIns;\n";
    const char comp[4] = {'x', 'y', 'z', 'w'};
    for (size_t n = 0; n < d.ins.size(); ++n) {
        const Instr& I = d.ins[n];
        const Block &A = d.L[0][I.a], &B = d.L[1][I.b], &O = d.L[2][I.o];
        const std::vector<IkPair>& P = pairs[n];
        const int D1 = A.d(), D3 = O.d(), np = (int)P.size(), nq = (np + 3) / 4;
        auto C = [&](int z) { std::ostringstream t; t << "c" << (z / 4) << "." << comp[z % 4]; return t.str(); };
        s << "template <> struct FIns<" << n << "> {\n";
        s << "  static constexpr int A = " << I.a << ", OB = " << I.o << ", XO = " << A.off / d.fast_U << ", GO = " << O.off / d.fast_U << ", Y0 = " << B.off
          << ", CY4 = " << cyoff[n] / 4 << ", WOFF = " << I.woff << ", D1 = " << D1 << ", D3 = " << D3 << ";\n";
        // ---- forward: FAST_CH channels per thread share the coefficient loads
        s << "  static OEQ_DEV void fwd(const T* x, const T4* cy, const T* w, T* acc) {\n";
        for (int q = 0; q < nq; ++q) s << "    const T4 c" << q << " = cy[CY4 + " << q << "];\n";
        s << "#pragma unroll\n    for (int ch = 0; ch < FAST_CH; ++ch) {\n";
        s << "      const T* xc = x + ch * D1; T* ac = acc + ch * FAST_GPC; const T wc = w[ch];\n";
        if (D1 <= D3) {
            for (int i = 0; i < D1; ++i) s << "      const T xs" << i << " = wc * xc[" << i << "];\n";
            for (int z = 0; z < np; ++z)
                s << "      ac[" << P[z].k << "] = oeq_fma(" << C(z) << ", xs" << P[z].i << ", ac[" << P[z].k << "]);\n";
        } else {
            for (int k = 0; k < D3; ++k) s << "      T t" << k << " = T(0);\n";
            for (int z = 0; z < np; ++z)
                s << "      t" << P[z].k << " = oeq_fma(" << C(z) << ", xc[" << P[z].i << "], t" << P[z].k << ");\n";
            for (int k = 0; k < D3; ++k) s << "      ac[" << k << "] = oeq_fma(wc, t" << k << ", ac[" << k << "]);\n";
        }
        s << "    }\n  }\n";
        // ---- fused second-order forward: acc += cy(y) . (w x2 + w2 x) + cy(y2) . (w x)
        if (dbl) {
            s << "  static OEQ_DEV void fwd3(const T* x, const T* x2, const T4* cy, const T4* cyb, const T* w, const T* w2, T* acc) {\n";
            for (int q = 0; q < nq; ++q) s << "    const T4 c" << q << " = cy[CY4 + " << q << "]; const T4 b" << q << " = cyb[CY4 + " << q << "];\n";
            s << "#pragma unroll\n    for (int ch = 0; ch < FAST_CH; ++ch) {\n";
            s << "      const T* xc = x + ch * D1; const T* yc = x2 + ch * D1; T* ac = acc + ch * FAST_GPC; const T wc = w[ch]; const T vc = w2[ch];\n";
            for (int i = 0; i < D1; ++i)
                s << "      const T xa" << i << " = oeq_fma(vc, xc[" << i << "], wc * yc[" << i << "]); const T xb" << i << " = wc * xc[" << i << "];\n";
            auto Bc = [&](int z) { std::ostringstream t; t << "b" << (z / 4) << "." << comp[z % 4]; return t.str(); };
            for (int z = 0; z < np; ++z)
                s << "      ac[" << P[z].k << "] = oeq_fma(" << C(z) << ", xa" << P[z].i << ", oeq_fma(" << Bc(z) << ", xb" << P[z].i << ", ac[" << P[z].k << "]));\n";
            s << "    }\n  }\n";
        }
        // ---- backward
        const bool scale_g = D3 <= D1;
        const int nqv = scale_g ? D3 : D1;
        s << "  static OEQ_DEV void bwd(const T* x, const T* g, const T4* cy, const T* w, const T* wdx, T* dx, T* dy, T* dw) {\n";
        for (int q = 0; q < nq; ++q) s << "    const T4 c" << q << " = cy[CY4 + " << q << "];\n";
        s << "    T qv[FAST_CH][" << nqv << "];\n";
        s << "#pragma unroll\n    for (int ch = 0; ch < FAST_CH; ++ch) {\n";
        s << "      const T* xc = x + ch * D1; const T* gc = g + ch * FAST_GPC; T* dxc = dx + ch * D1; const T wc = w[ch]; const T wx = wdx[ch];\n";
        for (int i = 0; i < D1; ++i) s << "      T s" << i << " = T(0);\n";
        for (int z = 0; z < np; ++z)
            s << "      s" << P[z].i << " = oeq_fma(" << C(z) << ", gc[" << P[z].k << "], s" << P[z].i << ");\n";
        s << "      T dwv = T(0);\n";
        for (int i = 0; i < D1; ++i) {
            s << "      dwv = oeq_fma(xc[" << i << "], s" << i << ", dwv);\n";
            s << "      dxc[" << i << "] = oeq_fma(wx, s" << i << ", dxc[" << i << "]);\n";
        }
        s << "      dw[ch] = dwv;\n";
        for (int t = 0; t < nqv; ++t) s << "      qv[ch][" << t << "] = wc * " << (scale_g ? "gc" : "xc") << "[" << t << "];\n";
        s << "    }\n";
        // dY: products are summed over the thread's channels before the fixed coefficients are applied
        std::vector<Nz> byik = I.nz;
        std::stable_sort(byik.begin(), byik.end(), [](const Nz& a, const Nz& b) { return a.i != b.i ? a.i < b.i : a.k < b.k; });
        for (size_t z = 0; z < byik.size();) {
            size_t m = z;
            s << "    { T pr = T(0);\n#pragma unroll\n      for (int ch = 0; ch < FAST_CH; ++ch) pr = oeq_fma(";
            if (scale_g) s << "x[ch * D1 + " << byik[z].i << "], qv[ch][" << byik[z].k << "]";
            else s << "qv[ch][" << byik[z].i << "], g[ch * FAST_GPC + " << byik[z].k << "]";
            s << ", pr);\n     ";
            while (m < byik.size() && byik[m].i == byik[z].i && byik[m].k == byik[z].k) {
                s << " dy[" << byik[m].j << "] = oeq_fma(T(" << hexf(byik[m].c) << "), pr, dy[" << byik[m].j << "]);";
                ++m;
            }
            s << " }\n";
            z = m;
        }
        s << "  }\n";
        // ---- fused second-order backward: s = cy(y).g and t = cy(y2).g;  dx += w2 s + w t;  dW = x2.s + x.t;
        //      dy[j] += C (w x2 + w2 x)[i] g[k]
        if (dbl) {
            s << "  static OEQ_DEV void bwd3(const T* x, const T* x2, const T* g, const T4* cy, const T4* cyb, const T* w, const T* w2, T* dx, T* dy, T* dw) {\n";
            for (int q = 0; q < nq; ++q) s << "    const T4 c" << q << " = cy[CY4 + " << q << "]; const T4 b" << q << " = cyb[CY4 + " << q << "];\n";
            auto Bc = [&](int z) { std::ostringstream t; t << "b" << (z / 4) << "." << comp[z % 4]; return t.str(); };
            s << "    T qv[FAST_CH][" << D1 << "];\n";
            s << "#pragma unroll\n    for (int ch = 0; ch < FAST_CH; ++ch) {\n";
            s << "      const T* xc = x + ch * D1; const T* yc = x2 + ch * D1; const T* gc = g + ch * FAST_GPC; T* dxc = dx + ch * D1; const T wc = w[ch]; const T vc = w2[ch];\n";
            for (int i = 0; i < D1; ++i) s << "      T s" << i << " = T(0), t" << i << " = T(0);\n";
            for (int z = 0; z < np; ++z)
                s << "      s" << P[z].i << " = oeq_fma(" << C(z) << ", gc[" << P[z].k << "], s" << P[z].i << "); t" << P[z].i << " = oeq_fma("
                  << Bc(z) << ", gc[" << P[z].k << "], t" << P[z].i << ");\n";
            s << "      T dwv = T(0);\n";
            for (int i = 0; i < D1; ++i) {
                s << "      dwv = oeq_fma(yc[" << i << "], s" << i << ", oeq_fma(xc[" << i << "], t" << i << ", dwv));\n";
                s << "      dxc[" << i << "] = oeq_fma(vc, s" << i << ", oeq_fma(wc, t" << i << ", dxc[" << i << "]));\n";
                s << "      qv[ch][" << i << "] = oeq_fma(vc, xc[" << i << "], wc * yc[" << i << "]);\n";
            }
            s << "      dw[ch] = dwv;\n    }\n";
            for (size_t z = 0; z < byik.size();) {
                size_t m = z;
                s << "    { T pr = T(0);\n#pragma unroll\n      for (int ch = 0; ch < FAST_CH; ++ch) pr = oeq_fma(qv[ch][" << byik[z].i
                  << "], g[ch * FAST_GPC + " << byik[z].k << "], pr);\n     ";
                while (m < byik.size() && byik[m].i == byik[z].i && byik[m].k == byik[z].k) {
                    s << " dy[" << byik[m].j << "] = oeq_fma(T(" << hexf(byik[m].c) << "), pr, dy[" << byik[m].j << "]);";
                    ++m;
                }
                s << " }\n";
                z = m;
            }
            s << "  }\n";
        }
        s << "};\n";
    }
    // Thread groups: with FAST_NG = 2 two sets of FU threads share an edge.  Backward: input blocks are dealt to the
    // groups (longest-processing-time first on CG nonzeros) so every dX block has one writer; forward: output blocks.
    {
        const int nb1 = (int)d.L[0].size(), nb3 = (int)d.L[2].size();
        std::vector<long> cost1(nb1, 0), cost3(nb3, 0);
        for (auto& I : d.ins) { cost1[I.a] += (long)I.nz.size() + 4; cost3[I.o] += (long)I.nz.size() + 4; }
        auto deal = [ng](const std::vector<long>& cost) {
            std::vector<int> order(cost.size()), grp(cost.size(), 0);
            for (size_t i = 0; i < order.size(); ++i) order[i] = (int)i;
            std::stable_sort(order.begin(), order.end(), [&](int a, int b) { return cost[a] > cost[b]; });
            long load[2] = {0, 0};
            for (int b : order) { const int g = (ng < 2 || load[0] <= load[1]) ? 0 : 1; grp[b] = g; load[g] += cost[b]; }
            return grp;
        };
        const std::vector<int> g1 = deal(cost1), g3 = deal(cost3);
        auto list = [&](const char* name, const std::vector<int>& v) {
            s << "constexpr int " << name << "[" << (v.empty() ? 1 : v.size()) << "] = {";
            for (size_t i = 0; i < v.size(); ++i) s << v[i] << (i + 1 < v.size() ? ", " : "");
            if (v.empty()) s << "0";
            s << "};\n";
        };
        s << "constexpr int FAST_NG = " << ng << ";\n";
        list("FP_X_OWNER", g1);   // backward: group that owns (reads X of, writes dX of) each input block
        list("FP_Z_OWNER", g3);   // forward: group that owns (accumulates, writes) each output block
        std::vector<int> needx0(nb1, 0), needx1(nb1, 0), needg0(nb3, 0), needg1(nb3, 0), gf, gb;
        for (auto& I : d.ins) {
            (g3[I.o] == 0 ? needx0 : needx1)[I.a] = 1;   // the instruction's forward group reads input block a
            (g1[I.a] == 0 ? needg0 : needg1)[I.o] = 1;   // the instruction's backward group reads gradient block o
            gf.push_back(g3[I.o]);
            gb.push_back(g1[I.a]);
        }
        list("FP_FWD_NEEDS_X0", needx0); list("FP_FWD_NEEDS_X1", needx1);
        list("FP_BWD_NEEDS_G0", needg0); list("FP_BWD_NEEDS_G1", needg1);
        list("FP_INS_GF", gf); list("FP_INS_GB", gb);
    }
    return s.str();
}

// Per-path tables for the tensor-core 'uvw' kernels (kernels/uvw_tc.cuh): paths ordered by the block they
// accumulate into, and for each path and component of that block the Clebsch-Gordan sum that produces one element of
// the A operand.
//   mode 0, forward:   z[b, o][w, k] = sum_p sum_u W_p[u, w] * (sum_{i,j} C[i,j,k] x[b, a][u, i] y[b][j])
//   mode 1, dx:       dx[b, a][u, i] = sum_p sum_w W_p[u, w] * (sum_{k,j} C[i,j,k] g[b, o][w, k] y[b][j])
// The second is the first with the roles of the input and output blocks exchanged and the weight block transposed, so
// the same kernel serves both from two sets of tables.
// A path of the tensor-core kernels: one 32 x 32 tile of an instruction's weight block (multiplicities are multiples of
// 32; the kernel weight order keeps such a tile contiguous: kernels/common.cuh::widx_uvw).
struct TcSub { int ins, uc, wc; };
std::vector<TcSub> tc_subpaths(const Desc& d) {
    std::vector<TcSub> subs;
    for (size_t n = 0; n < d.ins.size(); ++n)
        for (int uc = 0; uc < d.L[0][d.ins[n].a].mul / 32; ++uc)
            for (int wc = 0; wc < d.L[2][d.ins[n].o].mul / 32; ++wc) subs.push_back({(int)n, uc, wc});
    return subs;
}
int tc_sub_woff(const Desc& d, const TcSub& t) { return d.ins[t.ins].woff + t.uc * 32 * d.L[2][d.ins[t.ins].o].mul + t.wc * 1024; }

// Clebsch-Gordan terms of every instruction, by the component they produce: `by_i` = by component of the first input
// (gradient of x), else by output component.  TC_KBEG[8 n + k] .. TC_KBEG[8 n + k + 1] are the terms of instruction n.
void emit_tc_terms(std::ostringstream& s, const Desc& d, bool by_i, const char* prefix) {
    std::vector<long long> kbeg, ti, tj;
    std::vector<double> tcf;
    for (auto& I : d.ins) {
        const int dk = by_i ? d.L[0][I.a].d() : d.L[2][I.o].d();
        for (int k = 0; k < 8; ++k) {
            kbeg.push_back((long long)ti.size());
            if (k < dk)
                for (auto& z : I.nz)
                    if ((by_i ? z.i : z.k) == k) { ti.push_back(by_i ? z.k : z.i); tj.push_back(d.L[1][I.b].off + z.j); tcf.push_back(z.c); }
        }
    }
    kbeg.push_back((long long)ti.size());
    auto ilist = [&](const char* name, const std::vector<long long>& v) {
        s << "__constant__ int " << prefix << name << "[" << (v.empty() ? 1 : v.size()) << "] = {";
        for (size_t i = 0; i < v.size(); ++i) s << v[i] << (i + 1 < v.size() ? ", " : "");
        if (v.empty()) s << "0";
        s << "};\n";
    };
    ilist("KBEG", kbeg); ilist("TI", ti); ilist("TJ", tj);
    s << "__constant__ float " << prefix << "TC[" << (tcf.empty() ? 1 : tcf.size()) << "] = {";
    for (size_t i = 0; i < tcf.size(); ++i) s << hexf(tcf[i]) << (i + 1 < tcf.size() ? ", " : "");
    if (tcf.empty()) s << "0";
    s << "};\n";
}

std::string emit_tc_dw(const Desc& d);
std::string emit_tc(const Desc& d, int mode = 0) {
    std::ostringstream s;
    if (!d.tc) { s << "#define OEQ_TC 0\n"; return s.str(); }
    if (mode == 3) return emit_tc_dw(d);
    s << "#define OEQ_TC 1\n";
    const bool dx = mode == 1, dy = mode == 2;
    s << "#define TC_MODE " << mode << "\n";
    s << "#define TC_WT " << (mode != 0 ? 1 : 0) << "\n";
    s << "#define TC_KERNEL_NAME " << (dx ? "oeq_uvw_tc_backward_dx" : dy ? "oeq_uvw_tc_backward_dy" : "oeq_uvw_tc_forward") << "\n";
    s << "constexpr int TC_IN_DIM = " << (dx ? d.dim[2] : d.dim[0]) << ", TC_OUT_DIM = " << (dx ? d.dim[0] : d.dim[2]) << ";\n";
    const std::vector<TcSub> subs = tc_subpaths(d);
    // mode 2 (dy) accumulates nowhere across paths: every path is its own group; the paths are ordered by the input
    // tile they stage
    auto in_tile = [&](int q) { return d.ins[subs[q].ins].a * 64 + subs[q].uc; };
    auto out_tile = [&](int q) { return d.ins[subs[q].ins].o * 64 + subs[q].wc; };
    auto dst = [&](int q) { return dx ? in_tile(q) : dy ? q : out_tile(q); };   // tile the path accumulates into
    auto src = [&](int q) { return dx ? out_tile(q) : in_tile(q); };           // tile the path stages
    std::vector<int> order(subs.size());
    for (size_t i = 0; i < order.size(); ++i) order[i] = (int)i;
    std::stable_sort(order.begin(), order.end(), [&](int a, int b) { return dy ? src(a) < src(b) : dst(a) < dst(b); });
    // Inside a destination tile the order of the paths is free.  Paths that read the same tile are put next to each
    // other, and a group starts with the tile the previous group ended with where it can: the kernel keeps the
    // staged tile when the next path reads the same one.
    for (size_t g0 = 0; g0 < order.size();) {
        size_t g1 = g0;
        while (g1 < order.size() && dst(order[g1]) == dst(order[g0])) ++g1;
        std::stable_sort(order.begin() + g0, order.begin() + g1, [&](int a, int b) { return src(a) < src(b); });
        if (g0 > 0) {
            const int prev = src(order[g0 - 1]);
            std::stable_partition(order.begin() + g0, order.begin() + g1, [&](int q) { return src(q) == prev; });
        }
        g0 = g1;
    }
    std::vector<int> first(subs.size(), 0), last(subs.size(), 0);
    for (size_t q = 0; q < order.size(); ++q) {
        if (q == 0 || dst(order[q - 1]) != dst(order[q])) first[order[q]] = 1;
        if (q + 1 == order.size() || dst(order[q + 1]) != dst(order[q])) last[order[q]] = 1;
    }
    // run-time tables, one entry per path in schedule order
    auto ilist = [&](const char* name, const std::vector<long long>& v) {
        s << "__constant__ int " << name << "[" << (v.empty() ? 1 : v.size()) << "] = {";
        for (size_t i = 0; i < v.size(); ++i) s << v[i] << (i + 1 < v.size() ? ", " : "");
        if (v.empty()) s << "0";
        s << "};\n";
    };
    std::vector<long long> vd1, vd3, vx, vz, vw, vf, vl, vi;
    int maxd1 = 1;
    for (size_t q = 0; q < order.size(); ++q) {
        const TcSub& t = subs[order[q]];
        const Instr& I = d.ins[t.ins];
        const Block &A = d.L[0][I.a], &O = d.L[2][I.o];
        const Block &S = dx ? O : A, &D = dx ? A : O;   // block read, block accumulated into
        const int ts = dx ? t.wc : t.uc, td = dx ? t.uc : t.wc;
        vd1.push_back(S.d()); vd3.push_back(D.d());
        vx.push_back(S.off + ts * 32 * S.d()); vz.push_back(D.off + td * 32 * D.d()); vw.push_back(tc_sub_woff(d, t));
        vf.push_back(first[order[q]]); vl.push_back(last[order[q]]); vi.push_back(t.ins);
        if (S.d() > maxd1) maxd1 = S.d();
    }
    s << "constexpr int TC_MAXD1 = " << maxd1 << ", TC_NPATH = " << order.size() << ";\n";
    s << "constexpr int TC_XS2_D1 = " << tc_xs2_d1(d, mode, tc_smem_base_bytes(d, mode)) << ";\n";
    std::vector<long long> vnext(order.size(), -1);   // the next path of the schedule that stages another block
    for (size_t q = 0; q < order.size(); ++q)
        for (size_t r = q + 1; r < order.size(); ++r)
            if (vx[r] != vx[q]) { vnext[q] = (long long)r; break; }
    ilist("TC_NEXTX", vnext);
    ilist("TC_D1", vd1); ilist("TC_D3", vd3); ilist("TC_XOFF", vx); ilist("TC_ZOFF", vz); ilist("TC_WOFF", vw);
    ilist("TC_FIRST", vf); ilist("TC_LAST", vl); ilist("TC_INS", vi);
    emit_tc_terms(s, d, dx, "TC_");
    return s.str();
}

// Groups of the tensor-core weight-gradient kernel: paths (32 x 32 weight tiles) into the same tile of an output block, at
// most four per group and as many as have room for their staged input tiles (64 rows of 32 d1 + 8 floats each) beside
// the operand buffers.  Entries index tc_subpaths(d).
std::vector<std::vector<int>> tc_dw_groups(const Desc& d, size_t* xs_floats) {
    const size_t fixed = 4 * (size_t)(2 * 2 * 4096 + 2 * 2 * 1024 + 64 * (d.dim[1] | 1)) + 512;
    const size_t cap = (232448 - fixed) / 4 / 64;   // floats per staged row, summed over the slots
    const std::vector<TcSub> subs = tc_subpaths(d);
    auto rowlen = [&](int q) { return (size_t)(32 * d.L[0][d.ins[subs[q].ins].a].d() + 8); };
    std::vector<std::vector<int>> groups;
    size_t most = 0;
    for (size_t o = 0; o < d.L[2].size(); ++o)
        for (int wc = 0; wc < d.L[2][o].mul / 32; ++wc) {
            std::vector<int> cur;
            size_t used = 0;
            for (size_t q = 0; q < subs.size(); ++q)
                if (d.ins[subs[q].ins].o == (int)o && subs[q].wc == wc) {
                    if (!cur.empty() && (cur.size() == 4 || used + rowlen((int)q) > cap)) { groups.push_back(cur); cur.clear(); used = 0; }
                    cur.push_back((int)q);
                    used += rowlen((int)q);
                    most = std::max(most, used);
                }
            if (!cur.empty()) groups.push_back(cur);
        }
    if (xs_floats) *xs_floats = most * 64;
    return groups;
}
size_t tc_dw_smem_bytes(const Desc& d) {
    size_t xs_floats = 0;
    tc_dw_groups(d, &xs_floats);
    return std::max<size_t>(4 * (size_t)(2 * 2 * 4096 + 2 * 2 * 1024 + 64 * (d.dim[1] | 1) + xs_floats) + 512, 120 * 1024);
}

// Tables for the tensor-core weight-gradient kernel: the paths of an output tile in groups of up to four slots.
std::string emit_tc_dw(const Desc& d) {
    std::ostringstream s;
    s << "#define OEQ_TC 1\n#define TC_MODE 3\n#define TC_WT 0\n#define TC_KERNEL_NAME oeq_uvw_tc_unused\n";
    s << "constexpr int TC_IN_DIM = " << d.dim[0] << ", TC_OUT_DIM = " << d.dim[2] << ";\n";
    size_t xs_floats = 0;
    const std::vector<std::vector<int>> groups = tc_dw_groups(d, &xs_floats);
    const std::vector<TcSub> subs = tc_subpaths(d);
    auto ilist = [&](const char* name, const std::vector<long long>& v) {
        s << "__constant__ int " << name << "[" << (v.empty() ? 1 : v.size()) << "] = {";
        for (size_t i = 0; i < v.size(); ++i) s << v[i] << (i + 1 < v.size() ? ", " : "");
        if (v.empty()) s << "0";
        s << "};\n";
    };
    std::vector<long long> ns, gd3, gz, sd1, sx, sw, sxs, si;
    int maxd1 = 1;
    for (auto& grp : groups) {
        const TcSub& t0 = subs[grp[0]];
        const Block& O = d.L[2][d.ins[t0.ins].o];
        ns.push_back((long long)grp.size()); gd3.push_back(O.d()); gz.push_back(O.off + t0.wc * 32 * O.d());
        long long xsoff = 0;
        for (int slot = 0; slot < 4; ++slot) {
            const bool used = slot < (int)grp.size();
            const TcSub* t = used ? &subs[grp[slot]] : nullptr;
            const Block* A = used ? &d.L[0][d.ins[t->ins].a] : nullptr;
            sd1.push_back(used ? A->d() : 1); sx.push_back(used ? A->off + t->uc * 32 * A->d() : 0);
            sw.push_back(used ? tc_sub_woff(d, *t) : 0); si.push_back(used ? t->ins : -1);
            sxs.push_back(used ? xsoff : 0);
            if (used) { xsoff += 64LL * (32 * A->d() + 8); maxd1 = std::max(maxd1, A->d()); }
        }
    }
    s << "constexpr int TC_MAXD1 = " << maxd1 << ", TC_NPATH = 1, TC_XS2_D1 = 0;\n";
    s << "constexpr int TCW_NGRP = " << groups.size() << ";\n";
    s << "constexpr int TCW_XS_FLOATS = " << xs_floats << ";\n";
    ilist("TCW_XSOFF", sxs);
    ilist("TCW_NS", ns); ilist("TCW_D3", gd3); ilist("TCW_ZOFF", gz); ilist("TCW_D1", sd1); ilist("TCW_XOFF", sx);
    ilist("TCW_WOFF", sw); ilist("TCW_INS", si);
    emit_tc_terms(s, d, false, "TCW_");
    return s.str();
}

// --------------------------------------------------------------------------------------- kernel families
enum Family {
    FAM_GENERIC = 0,
    FAM_FAST_FWD_TP, FAM_FAST_FWD_DET, FAM_FAST_FWD_ATOMIC, FAM_FAST_BWD_TP, FAM_FAST_BWD_DET, FAM_FAST_BWD_ATOMIC,
    FAM_FAST_SCATTER,
    FAM_FAST_BWD2_TP, FAM_FAST_BWD2_DET, FAM_FAST_BWD2_ATOMIC,   // second-order variants of the backward kernels
    FAM_UVW_TC,                                                  // tcgen05 'uvw' forward
    FAM_FAST_FWD3_TP, FAM_FAST_FWD3_DET,                         // fused second-order forward (three terms in one pass)
    FAM_UVW_TC_DX, FAM_UVW_TC_DY, FAM_UVW_TC_DW,                 // tcgen05 'uvw' backward: gradients of x, y and the weights
    FAM_COUNT
};
const char* const kFamilyNames[FAM_COUNT] = {"generic", "fast_fwd_tp", "fast_fwd_det", "fast_fwd_atomic", "fast_bwd_tp",
                                             "fast_bwd_det", "fast_bwd_atomic", "fast_scatter", "fast_bwd2_tp",
                                             "fast_bwd2_det", "fast_bwd2_atomic", "uvw_tc", "fast_fwd3_tp", "fast_fwd3_det",
                                             "uvw_tc_dx", "uvw_tc_dy", "uvw_tc_dw"};
const char* family_name(int f) { return (f >= 0 && f < FAM_COUNT) ? kFamilyNames[f] : "?"; }
int family_from_name(const std::string& n) {
    for (int f = 0; f < FAM_COUNT; ++f)
        if (n == kFamilyNames[f]) return f;
    if (n == "generic_forward" || n == "generic_backward") return FAM_GENERIC;
    return -1;
}

// Edge streams per CTA for a kernel family: the first-order kernels except the atomic forward (whose staged output
// row leaves no room for three rings); 1 when the problem or the caller rules them out.
int family_streams(const Desc& d, int fam, bool allow) {
    const bool eligible = ((fam == FAM_FAST_FWD_TP || fam == FAM_FAST_FWD_DET) && g_streams_fwd) || fam == FAM_FAST_BWD_TP ||
                          fam == FAM_FAST_BWD_DET || fam == FAM_FAST_BWD_ATOMIC;
    return (allow && eligible && d.fast && d.fast_V > 1) ? d.fast_V : 1;
}

std::string family_source(const Desc& d, const std::string& header, int fam, bool allow_streams = true) {
    std::string src = header;
    if (fam == FAM_GENERIC) {
        src += K_COMMON;
        src += K_GENERIC;
    } else if (fam == FAM_UVW_TC || (fam >= FAM_UVW_TC_DX && fam <= FAM_UVW_TC_DW)) {
        src += emit_tc(d, fam == FAM_UVW_TC ? 0 : fam - FAM_UVW_TC_DX + 1);
        src += K_COMMON;
        src += K_UVW_TC;
    } else {
        // Forward kernels carry two channels per thread in two block-owning groups (their code is small enough to stay
        // in the instruction cache); the backward kernels, three times larger, keep one channel per thread and one
        // code stream, which measured faster than the split variants (those stalled on instruction fetch).
        const bool fwd3 = fam == FAM_FAST_FWD3_TP || fam == FAM_FAST_FWD3_DET;
        const bool fwd = fwd3 || (fam >= FAM_FAST_FWD_TP && fam <= FAM_FAST_FWD_ATOMIC);
        const bool dbl = fwd3 || (fam >= FAM_FAST_BWD2_TP && fam <= FAM_FAST_BWD2_ATOMIC);
        const int V = family_streams(d, fam, allow_streams);
        const bool bwd1 = !fwd && !dbl;   // first-order backward: its own stage count and residency
        const int stages = V > 1 ? d.fast_SV : dbl ? d.fast_S4 : (fam == FAM_FAST_FWD_ATOMIC ? d.fast_S3 : bwd1 ? d.fastb_S : d.fast_S);
        const size_t smem = V > 1 ? d.fast_smemV : dbl ? d.fast_smem4 : (fam == FAM_FAST_FWD_ATOMIC ? d.fast_smem3 : bwd1 ? d.fastb_smem : d.fast_smem);
        src += emit_fast(d, fwd ? d.fast_ch : 1, fwd ? d.fast_ng : d.fast_bwd_ng, dbl, stages, smem, V, bwd1 ? d.fastb_ctas : d.fast_ctas);
        // the second-order variants reuse the backward entry points (kernel ids 3..5)
        src += "#define FAST_KERNEL " + std::to_string(fwd3 ? fam - FAM_FAST_FWD3_TP : dbl ? fam - FAM_FAST_BWD2_TP + 3 : fam - FAM_FAST_FWD_TP) + "\n";
        src += K_COMMON;   // (FAST_KERNEL is defined before the kernel file: it sizes the shared-memory layout)
        src += K_FAST_UVU;
    }
    return src;
}

// -------------------------------------------------------------------------------------- NVRTC + caching
uint64_t fnv1a(const std::string& s) {
    uint64_t h = 1469598103934665603ull;
    for (unsigned char c : s) { h ^= c; h *= 1099511628211ull; }
    return h;
}

std::string default_cache_dir() {
    if (const char* e = getenv("OEQB_CACHE_DIR")) return e;
    Dl_info info;
    if (dladdr((void*)&default_cache_dir, &info) && info.dli_fname) {
        std::string p = info.dli_fname;
        size_t slash = p.find_last_of('/');
        if (slash != std::string::npos) return p.substr(0, slash) + "/_cubin_cache";
    }
    return "/tmp/oeq_b200_cubin_cache";
}

const std::string& cache_dir() {
    if (g_cache_dir.empty()) g_cache_dir = default_cache_dir();
    return g_cache_dir;
}

bool read_file(const std::string& path, std::string& out) {
    FILE* f = fopen(path.c_str(), "rb");
    if (!f) return false;
    fseek(f, 0, SEEK_END);
    long n = ftell(f);
    fseek(f, 0, SEEK_SET);
    out.resize(n > 0 ? n : 0);
    size_t got = n > 0 ? fread(&out[0], 1, n, f) : 0;
    fclose(f);
    return got == (size_t)(n > 0 ? n : 0) && n > 0;
}

void write_file_atomic(const std::string& path, const std::string& data) {
    mkdir(cache_dir().c_str(), 0755);
    std::string tmp = path + ".tmp" + std::to_string((long long)getpid());
    FILE* f = fopen(tmp.c_str(), "wb");
    if (!f) return;
    size_t put = fwrite(data.data(), 1, data.size(), f);
    fclose(f);
    if (put == data.size()) rename(tmp.c_str(), path.c_str()); else remove(tmp.c_str());
}

// Compiles `src` for sm_100a; returns the cubin (from the disk cache when present).
// *from_cache (optional) receives the cache file's path when the cubin was read from it, "" when it was compiled now.
int compile_cubin(const std::string& src, const char* label, std::string& cubin, std::string* from_cache = nullptr) {
    if (from_cache) from_cache->clear();
    static const char* opts[] = {"--gpu-architecture=sm_100a", "--std=c++17", "-lineinfo", "-default-device",
                                 "--extra-device-vectorization"};
    const int nopts = sizeof(opts) / sizeof(opts[0]);
    int major = 0, minor = 0;
    nvrtcVersion(&major, &minor);
    std::string keytext = src;
    for (int i = 0; i < nopts; ++i) keytext += opts[i];
    keytext += std::to_string(major * 100 + minor);
    char name[64];
    snprintf(name, sizeof name, "/%016llx.cubin", (unsigned long long)fnv1a(keytext));
    const std::string path = cache_dir() + name;
    if (read_file(path, cubin)) {
        if (g_log) fprintf(stderr, "[oeq_b200] %s: cubin cache hit %s\n", label, path.c_str());
        if (from_cache) *from_cache = path;
        return OEQB_OK;
    }
    nvrtcProgram prog;
    nvrtcResult r = nvrtcCreateProgram(&prog, src.c_str(), label, 0, nullptr, nullptr);
    if (r != NVRTC_SUCCESS) return fail(OEQB_ECOMPILE, "nvrtcCreateProgram: %s", nvrtcGetErrorString(r));
    r = nvrtcCompileProgram(prog, nopts, opts);
    if (r != NVRTC_SUCCESS) {
        size_t ls = 0;
        nvrtcGetProgramLogSize(prog, &ls);
        std::string log(ls, '\0');
        if (ls) nvrtcGetProgramLog(prog, &log[0]);
        nvrtcDestroyProgram(&prog);
        if (log.size() > 3500) log.resize(3500);
        return fail(OEQB_ECOMPILE, "NVRTC failed for %s: %s\n%s", label, nvrtcGetErrorString(r), log.c_str());
    }
    size_t cs = 0;
    nvrtcGetCUBINSize(prog, &cs);
    cubin.resize(cs);
    nvrtcGetCUBIN(prog, &cubin[0]);
    nvrtcDestroyProgram(&prog);
    write_file_atomic(path, cubin);
    if (g_log) fprintf(stderr, "[oeq_b200] %s: compiled %zu bytes of cubin\n", label, cs);
    return OEQB_OK;
}

struct Program {
    cudaLibrary_t lib = nullptr;
    std::map<std::string, cudaKernel_t> kernels;
    std::map<std::string, int> smem_set;  // kernel -> bitmask of devices whose smem attribute was raised
    std::string cubin;                    // kept alive for lazy per-context loading
    bool regs_checked = false;            // multi-stream kernels: register count verified against the hand-over scheme
};

struct Entry {
    Desc d;
    uint64_t desc_hash = 0;     // of the descriptor text this entry was built from: a key reused for another problem is refused
    size_t desc_len = 0;
    const void* seen_ptr = nullptr;   // last caller buffer whose contents were compared (callers pass the same buffer again)
    std::string header;
    std::unique_ptr<Program> prog[FAM_COUNT];
    std::unique_ptr<Program> prog_single[FAM_COUNT];   // the same families built with one edge stream per CTA
    bool streams_off = false;                           // a multi-stream kernel came out with the wrong register count
};

std::map<int64_t, std::unique_ptr<Entry>> g_entries;

// Caller holds g_mutex.
int get_entry(const void* desc, size_t len, int64_t key, Entry** out) {
    auto it = g_entries.find(key);
    if (it != g_entries.end()) {
        Entry* have = it->second.get();
        if (desc && len > 0 && !(desc == have->seen_ptr && len == have->desc_len)) {
            if (len != have->desc_len || fnv1a(std::string((const char*)desc, len)) != have->desc_hash)
                return fail(OEQB_EINVAL, "key %lld was first used with a different descriptor: keys must identify one problem",
                            (long long)key);
            have->seen_ptr = desc;
        }
        *out = have;
        return OEQB_OK;
    }
    if (!desc || len == 0) return fail(OEQB_EINVAL, "descriptor is empty");
    auto e = std::make_unique<Entry>();
    e->desc_hash = fnv1a(std::string((const char*)desc, len));
    e->desc_len = len;
    e->seen_ptr = desc;
    std::string why;
    if (!parse_desc((const char*)desc, len, e->d, why)) return fail(OEQB_EPARSE, "descriptor: %s", why.c_str());
    e->header = emit_header(e->d);
    *out = e.get();
    g_entries[key] = std::move(e);
    return OEQB_OK;
}

// Caller holds g_mutex.
int get_program(Entry* e, int fam, Program** out, bool allow_streams = true) {
    std::unique_ptr<Program>& slot = allow_streams ? e->prog[fam] : e->prog_single[fam];
    if (slot) { *out = slot.get(); return OEQB_OK; }
    auto p = std::make_unique<Program>();
    const std::string src = family_source(e->d, e->header, fam, allow_streams);
    std::string cache_path;
    int rc = compile_cubin(src, family_name(fam), p->cubin, &cache_path);
    if (rc) return rc;
    cudaError_t ce = cudaLibraryLoadData(&p->lib, p->cubin.data(), nullptr, nullptr, 0, nullptr, nullptr, 0);
    if (ce != cudaSuccess && !cache_path.empty()) {
        // a truncated or foreign file in the cache: drop it and compile afresh, once
        cudaGetLastError();
        remove(cache_path.c_str());
        if (g_log) fprintf(stderr, "[oeq_b200] %s: cached cubin %s did not load (%s); recompiling\n", family_name(fam),
                           cache_path.c_str(), cudaGetErrorString(ce));
        if ((rc = compile_cubin(src, family_name(fam), p->cubin, nullptr))) return rc;
        ce = cudaLibraryLoadData(&p->lib, p->cubin.data(), nullptr, nullptr, 0, nullptr, nullptr, 0);
    }
    if (ce != cudaSuccess) return fail(OEQB_ECOMPILE, "cudaLibraryLoadData(%s): %s", family_name(fam), cudaGetErrorString(ce));
    *out = p.get();
    slot = std::move(p);
    return OEQB_OK;
}

int get_kernel(Program* p, const char* name, size_t smem, cudaKernel_t* out) {
    auto it = p->kernels.find(name);
    if (it == p->kernels.end()) {
        cudaKernel_t k;
        cudaError_t ce = cudaLibraryGetKernel(&k, p->lib, name);
        if (ce != cudaSuccess) return fail(OEQB_ECOMPILE, "kernel %s not found: %s", name, cudaGetErrorString(ce));
        it = p->kernels.emplace(name, k).first;
    }
    if (smem > 48 * 1024) {
        int dev = 0;
        CUDA_TRY(cudaGetDevice(&dev));
        int& mask = p->smem_set[name];
        if (!(mask & (1 << dev))) {
            CUDA_TRY(cudaFuncSetAttribute((const void*)it->second, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem));
            mask |= 1 << dev;
        }
    }
    *out = it->second;
    return OEQB_OK;
}

int launch(cudaKernel_t k, unsigned grid, unsigned block, size_t smem, void** args, cudaStream_t st) {
    cudaError_t ce = cudaLaunchKernel((const void*)k, dim3(grid), dim3(block), args, smem, st);
    if (ce != cudaSuccess) return fail(OEQB_ECUDA, "kernel launch failed: %s", cudaGetErrorString(ce));
    g_launches.fetch_add(1, std::memory_order_relaxed);
    return OEQB_OK;
}

int sm_count() {
    static int cached[64] = {0};
    int dev = 0;
    if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= 64) return 148;
    if (!cached[dev]) {
        int n = 0;
        if (cudaDeviceGetAttribute(&n, cudaDevAttrMultiProcessorCount, dev) != cudaSuccess || n <= 0) n = 148;
        cached[dev] = n;
    }
    return cached[dev];
}

// ------------------------------------------------------------------------------------------ generic path
struct FwdParams {
    const void* x; const void* y; const void* W; void* z;
    const void* rows; const void* cols;
    long long n_units; long long n_edges;
    int unit_mode; int out_mode;
};
struct BwdParams {
    const void* x; const void* y_dx; const void* y_dw; const void* W; const void* g;
    void* dx; void* dy; void* dW;
    const void* rows; const void* cols; const void* perm;
    long long n_units; long long n_edges;
    int unit_mode; int accum;
    void* dW_part;
};
enum { UNIT_ITEM = 0, UNIT_EDGE = 1, UNIT_SEGMENT = 2 };
enum { OUT_STORE = 0, OUT_ADD = 1, OUT_ATOMIC = 2 };

unsigned generic_grid(long long units) {
    long long want = (units + 3) / 4;  // 4 warps per block
    long long cap = (long long)sm_count() * 16;
    if (want < 1) want = 1;
    return (unsigned)(want < cap ? want : cap);
}

int generic_forward(Entry* e, FwdParams p, cudaStream_t st) {
    if (p.n_units <= 0) return OEQB_OK;
    Program* prog;
    int rc = get_program(e, FAM_GENERIC, &prog);
    if (rc) return rc;
    cudaKernel_t k;
    if ((rc = get_kernel(prog, "oeq_generic_forward", 0, &k))) return rc;
    void* args[] = {&p};
    return launch(k, generic_grid(p.n_units), 128, 0, args, st);
}

int keep_pool_memory();

int generic_backward(Entry* e, BwdParams p, cudaStream_t st) {
    if (p.n_units <= 0) return OEQB_OK;
    Program* prog;
    int rc = get_program(e, FAM_GENERIC, &prog);
    if (rc) return rc;
    if (e->d.shared && p.unit_mode != UNIT_SEGMENT) {
        // shared weights: path-major kernel that sums dW over a chunk of items in registers and stores the chunk's sums
        // as one row of a partials matrix; a second kernel adds the rows in chunk order, so dW is bitwise reproducible
        // (the chunking does not depend on the grid).  The matrix lives in stream-ordered scratch for the call.
        // The kernel adds to dX, so for the tensor product dX has to start at zero (the convolution zeroes it anyway).
        const Desc& d = e->d;
        if (p.unit_mode == UNIT_ITEM && !p.accum)
            CUDA_TRY(cudaMemsetAsync(p.dx, 0, (size_t)p.n_edges * d.dim[0] * d.elt(), st));
        cudaKernel_t ks, kr;
        if ((rc = get_kernel(prog, "oeq_generic_backward_shared", 0, &ks))) return rc;
        if ((rc = get_kernel(prog, "oeq_generic_dw_reduce", 0, &kr))) return rc;
        int chunk = 32;
        long long chunks = (p.n_edges + chunk - 1) / chunk;
        void* part = nullptr;
        if ((rc = keep_pool_memory())) return rc;
        CUDA_TRY(cudaMallocAsync(&part, (size_t)chunks * d.wn * d.elt(), st));
        p.dW_part = part;
        void* args[] = {&p, &chunk};
        rc = launch(ks, generic_grid(chunks), 128, 0, args, st);
        if (!rc) {
            // the entry points zero dW before the first pass, so the reduce always adds to what is there
            int accum = 1;
            void* rargs[] = {&part, &chunks, &p.dW, &accum};
            rc = launch(kr, (unsigned)((d.wn + 31) / 32), 256, 0, rargs, st);
        }
        cudaFreeAsync(part, st);
        return rc;
    }
    cudaKernel_t k;
    if ((rc = get_kernel(prog, "oeq_generic_backward", 0, &k))) return rc;
    void* args[] = {&p};
    return launch(k, generic_grid(p.n_units), 128, 0, args, st);
}

// ------------------------------------------------------------------------------- channel-parallel path
struct FastParams {
    const void* X; const void* Y; const void* W; const void* G;
    void* Z; void* dX; void* dY; void* dW; void* scratch;
    const void* rows; const void* cols;
    long long N; long long E;
    int* status;
    int accum;         // forward kernels: add to the output rows instead of overwriting them
    int pad;
    const void* X2; const void* Y2; const void* W2;   // fused second-order forward
    const void* eorder;                               // unsorted edge lists: position -> edge id, grouped by receiver
};

constexpr size_t kAlign = 256;
size_t round_up(size_t v) { return (v + kAlign - 1) / kAlign * kAlign; }

// One host-mapped status word per device: kernels store a non-zero code when a bounded wait runs out.
int* g_status_host[64] = {nullptr};
int* g_status_dev[64] = {nullptr};

int status_word(int** dev_ptr) {
    int dev = 0;
    CUDA_TRY(cudaGetDevice(&dev));
    if (dev < 0 || dev >= 64) return fail(OEQB_EINVAL, "device index %d out of range", dev);
    if (!g_status_host[dev]) {
        int* h = nullptr;
        CUDA_TRY(cudaHostAlloc((void**)&h, 64, cudaHostAllocMapped));
        memset(h, 0, 64);
        int* dptr = nullptr;
        CUDA_TRY(cudaHostGetDevicePointer((void**)&dptr, h, 0));
        g_status_host[dev] = h;
        g_status_dev[dev] = dptr;
    }
    const int code = *(volatile int*)g_status_host[dev];
    if (code != 0) {
        *(volatile int*)g_status_host[dev] = 0;
        if (code == gprep::STATUS_BAD_INDEX)
            return fail(OEQB_EINVAL, "an earlier call was given an index array (rows / cols / transpose_perm) with a value "
                                     "out of range, or a receiver list that is not sorted; its outputs are invalid");
        return fail(OEQB_EKERNEL, "an earlier kernel gave up a bounded wait (code %d); its outputs are invalid", code);
    }
    if (dev_ptr) *dev_ptr = g_status_dev[dev];
    return OEQB_OK;
}

// Groups an unsorted edge list by receiver into ws (layout: [order: E indices][scratch of the grouping]); *order receives
// the position -> edge id list.  Returns OEQB_OK, or a negative number when the workspace is too small (the caller then
// takes the path that needs none).
size_t atomic_order_bytes(const Desc& d, long long N, long long E) {
    return round_up((size_t)(E > 0 ? E : 1) * (d.idx == 3 ? 4 : 8)) + gprep::group_workspace_bytes(N, E);
}
int group_by_receiver(const Desc& d, long long N, long long E, const void* rows, void* ws, long long ws_bytes,
                      cudaStream_t st, const void** order) {
    if (!ws || ws_bytes < (long long)atomic_order_bytes(d, N, E) || ((uintptr_t)ws & 15u)) return -1;
    int* status = nullptr;
    if (int rc = status_word(&status)) return rc;
    void* scratch = (char*)ws + round_up((size_t)E * (d.idx == 3 ? 4 : 8));
    long long launches = 0;
    bool ok;
    if (d.idx == 3) ok = gprep::group_by_key<int>((const int*)rows, nullptr, E, N, (int*)ws, nullptr, nullptr, scratch, status, st, nullptr, &launches);
    else ok = gprep::group_by_key<long long>((const long long*)rows, nullptr, E, N, (long long*)ws, nullptr, nullptr, scratch, status, st, nullptr, &launches);
    g_launches.fetch_add(launches, std::memory_order_relaxed);
    if (!ok) return fail(OEQB_ECUDA, "grouping the edge list by receiver failed: %s", cudaGetErrorString(cudaGetLastError()));
    *order = ws;
    return OEQB_OK;
}

bool aligned16(std::initializer_list<const void*> ptrs) {
    for (const void* p : ptrs)
        if (((uintptr_t)p & 15u) != 0) return false;
    return true;
}

bool use_fast(const Desc& d) { return d.fast && !g_force_generic; }


// kernel: 0 fwd_tp, 1 fwd_det, 2 fwd_atomic, 3 bwd_tp, 4 bwd_det, 5 bwd_atomic
int fast_launch(Entry* e, int kernel, FastParams p, cudaStream_t st, int* status_override = nullptr, bool dbl = false) {
    static const char* names1[6] = {"oeq_fast_forward_tp", "oeq_fast_forward_det", "oeq_fast_forward_atomic",
                                    "oeq_fast_backward_tp", "oeq_fast_backward_det", "oeq_fast_backward_atomic"};
    static const char* names2[6] = {"oeq_fast_double_backward_A_tp", "oeq_fast_double_backward_A_det", "",
                                    "oeq_fast_double_backward_B_tp", "oeq_fast_double_backward_B_det",
                                    "oeq_fast_double_backward_B_atomic"};
    const char* const* names = dbl ? names2 : names1;
    const Desc& d = e->d;
    int rc;
    if (status_override) p.status = status_override;
    else if ((rc = status_word(&p.status))) return rc;
    Program* prog;
    const bool fwd3 = dbl && kernel < 2;   // fused second-order forward (batch and sorted-convolution variants)
    const int fam = fwd3 ? FAM_FAST_FWD3_TP + kernel : dbl ? FAM_FAST_BWD2_TP + (kernel - 3) : FAM_FAST_FWD_TP + kernel;
    cudaKernel_t k;
    int V = family_streams(d, fam, !e->streams_off);
    if (V > 1) {
        // One CTA per SM with V consumer warpgroups and a producer warpgroup that hands registers over (setmaxnreg).
        // The hand-over only balances when the launch allocates exactly 65536 / threads registers per thread: a kernel
        // compiled to anything else is not used (its consumers would wait for registers that are never released).
        if ((rc = get_program(e, fam, &prog, true))) return rc;
        if ((rc = get_kernel(prog, names[kernel], d.fast_smemV, &k))) return rc;
        if (!prog->regs_checked) {
            cudaFuncAttributes attr;
            CUDA_TRY(cudaFuncGetAttributes(&attr, (const void*)k));
            const int threads = V * 128 + 128, want = 65536 / threads / 8 * 8;
            prog->regs_checked = true;
            if (attr.numRegs != want || attr.maxThreadsPerBlock < threads) {
                if (g_log) fprintf(stderr, "[oeq_b200] %s: multi-stream kernel has %d registers (%d needed); using the "
                                           "two-CTA variant\n", family_name(fam), attr.numRegs, want);
                e->streams_off = true;
                V = 1;
            }
        }
    }
    if (V > 1) {
        long long grid = sm_count();
        const long long work = ((p.E > 0 ? p.E : 1) + V - 1) / V;
        if (grid > work) grid = work;
        void* args[] = {&p};
        return launch(k, (unsigned)grid, (unsigned)(V * 128 + 128), d.fast_smemV, args, st);
    }
    const bool bwd1 = kernel >= 3 && !dbl;   // first-order backward: its own stage count and residency
    const size_t smem = dbl ? d.fast_smem4 : (kernel == 2 ? d.fast_smem3 : bwd1 ? d.fastb_smem : d.fast_smem);
    if ((rc = get_program(e, fam, &prog, false))) return rc;
    if ((rc = get_kernel(prog, names[kernel], smem, &k))) return rc;
    long long grid = (long long)sm_count() * (bwd1 ? d.fastb_ctas : d.fast_ctas);
    const long long work = p.E > 0 ? p.E : 1;
    if (grid > work) grid = work;
    void* args[] = {&p};
    const unsigned consumers = kernel < 3 ? (unsigned)(d.fast_ng * d.fast_U / d.fast_ch) : (unsigned)(d.fast_bwd_ng * d.fast_U);
    const int producers = fast_producers(dbl ? d.fast_S4 : (kernel == 2 ? d.fast_S3 : bwd1 ? d.fastb_S : d.fast_S));
    return launch(k, (unsigned)grid, consumers + 32 * producers, smem, args, st);
}

// dX[c] = sum of the per-edge rows in scratch over the sender's edges, in sender-major list order.  Two steps: the sender
// offsets (once), then the row sums for a range of senders [c_begin, c_end).
int fast_scatter_offsets(Entry* e, const void* cols, const void* perm, long long N, long long E, void* colptr, cudaStream_t st) {
    int rc;
    Program* prog;
    if ((rc = get_program(e, FAM_FAST_SCATTER, &prog))) return rc;
    cudaKernel_t k1;
    if ((rc = get_kernel(prog, "oeq_fixup_backward_offsets", 0, &k1))) return rc;
    void* args[] = {(void*)&cols, (void*)&perm, &E, &N, &colptr};
    return launch(k1, (unsigned)((E + 1 + 255) / 256), 256, 0, args, st);
}

int fast_scatter_rows(Entry* e, const void* scratch, const void* perm, const void* colptr, long long c_begin, long long c_end,
                      void* dX, cudaStream_t st) {
    if (c_end <= c_begin) return OEQB_OK;
    int rc;
    Program* prog;
    if ((rc = get_program(e, FAM_FAST_SCATTER, &prog))) return rc;
    cudaKernel_t k2;
    if ((rc = get_kernel(prog, "oeq_fixup_backward_reduce", 0, &k2))) return rc;
    long long grid = (long long)sm_count() * 8;
    if (grid > c_end - c_begin) grid = c_end - c_begin;
    void* args[] = {(void*)&scratch, (void*)&perm, (void*)&colptr, &c_begin, &c_end, &dX};
    return launch(k2, (unsigned)grid, 256, 0, args, st);
}

int fast_scatter(Entry* e, const void* scratch, const void* cols, const void* perm, long long N, long long E, void* colptr,
                 void* dX, cudaStream_t st) {
    if (int rc = fast_scatter_offsets(e, cols, perm, N, E, colptr, st)) return rc;
    return fast_scatter_rows(e, scratch, perm, colptr, 0, N, dX, st);
}

// ------------------------------------------------------------------- scratch that nobody has to allocate
// Backing store of oeqb_conv_backward_noalloc: a fixed array that is part of the library image, so every GPU that
// loads the library holds these bytes until the process exits.  In host code the name below is only a handle for
// the symbol; the device address is looked up once per device with cudaGetSymbolAddress.
static __device__ __align__(256) unsigned char g_noalloc_scratch[OEQB_NOALLOC_SCRATCH_BYTES];
void* g_noalloc_ptr[64] = {nullptr};

int noalloc_scratch(void** out) {
    int dev = 0;
    CUDA_TRY(cudaGetDevice(&dev));
    if (dev < 0 || dev >= 64) return fail(OEQB_EINVAL, "device index %d out of range", dev);
    if (!g_noalloc_ptr[dev]) {
        void* p = nullptr;
        cudaError_t ce = cudaGetSymbolAddress(&p, g_noalloc_scratch);
        if (ce != cudaSuccess || !p)
            return fail(OEQB_ECUDA, "cudaGetSymbolAddress(built-in scratch) failed on device %d: %s", dev, cudaGetErrorString(ce));
        g_noalloc_ptr[dev] = p;
    }
    *out = g_noalloc_ptr[dev];
    return OEQB_OK;
}

// ------------------------------------------------------------------------------------ tensor-core 'uvw'
struct TcParams {
    const void* x; const void* y; const void* W; void* z;
    const void* g;
    long long batch;
    int accum;
    int* status;
};
struct TcDwParams {
    const void* x; const void* y; const void* g; void* part;
    long long batch;
    int grp_begin, grp_end;
    int* status;
};
// sizeof(TcShared) in kernels/uvw_tc.cuh, rounded up: operand buffers + staged block + harmonics (+ the dy partials);
// mode as in emit_tc
// Components of the largest block the second staging buffer of the forward / dx kernels can hold beside everything else
// (0: no second buffer); `base` is the shared memory the kernel needs without it.
int tc_xs2_d1(const Desc& d, int mode, size_t base) {
    if (mode == 2) return 0;
    int maxd1 = 1;
    for (auto& I : d.ins) maxd1 = std::max(maxd1, mode == 1 ? d.L[2][I.o].d() : d.L[0][I.a].d());
    for (int dd = maxd1; dd >= 1; dd -= 2)
        if (base + 4 * (size_t)128 * (32 * dd + 4) <= 232448) return dd;
    return 0;
}

size_t tc_smem_base_bytes(const Desc& d, int mode);
size_t tc_smem_bytes(const Desc& d, int mode) {
    const size_t base = tc_smem_base_bytes(d, mode);
    const int d2 = tc_xs2_d1(d, mode, base);
    // never less than half of an SM's shared memory: a CTA allocates all of the tensor memory, so only one may be resident
    return std::max<size_t>(base + (d2 > 0 ? 4 * (size_t)128 * (32 * d2 + 4) : 0), 120 * 1024);
}
size_t tc_smem_base_bytes(const Desc& d, int mode) {   // without the second staging buffer (for tc_xs2_d1)
    int maxd1 = 1;
    for (auto& I : d.ins) maxd1 = std::max(maxd1, mode == 1 ? d.L[2][I.o].d() : d.L[0][I.a].d());
    const size_t dys = mode == 2 ? 512 * (size_t)(d.dim[1] | 1) : 4;
    const size_t ys = mode == 2 ? 4 : 128 * (size_t)(((int)d.dim[1] + 3) & ~3);
    const size_t xs = 128 * (size_t)(32 * maxd1 + (mode == 2 ? 1 : 4));
    return 4 * (2 * 2 * 4096 + 2 * 2 * 1024 + xs + ys + dys) + 256;
}

// mode 0: z from (x, y, W); mode 1: the gradient of x from (g, y, W), passed in the places of x and z; mode 2: the
// gradient of y (in the place of z) from (x, W, g)
int tc_forward(Entry* e, TcParams p, cudaStream_t st, int mode = 0) {
    static const char* names[3] = {"oeq_uvw_tc_forward", "oeq_uvw_tc_backward_dx", "oeq_uvw_tc_backward_dy"};
    int rc;
    if (!p.accum && ((mode == 0 && e->d.tc_zero_z) || (mode == 1 && e->d.tc_zero_dx)))
        CUDA_TRY(cudaMemsetAsync(p.z, 0, (size_t)p.batch * e->d.dim[mode == 0 ? 2 : 0] * sizeof(float), st));
    if ((rc = status_word(&p.status))) return rc;
    Program* prog;
    if ((rc = get_program(e, mode == 0 ? FAM_UVW_TC : FAM_UVW_TC_DX + (mode - 1), &prog))) return rc;
    cudaKernel_t k;
    const size_t smem = e->d.tc_smem[mode];
    if ((rc = get_kernel(prog, names[mode], smem, &k))) return rc;
    long long tiles = (p.batch + 127) / 128, grid = sm_count();
    if (grid > tiles) grid = tiles;
    void* args[] = {&p};
    return launch(k, (unsigned)grid, 16 * 32 + 32, smem, args, st);   // TC_THREADS: sixteen compute warps + the issuing warp
}

// Keep freed stream-ordered scratch in the device's pool: by default the pool gives memory back to the driver at every
// synchronisation and the next call pays for mapping it again.
int keep_pool_memory() {
    static bool pool_kept[64] = {false};
    int dev = 0;
    CUDA_TRY(cudaGetDevice(&dev));
    if (dev >= 0 && dev < 64 && !pool_kept[dev]) {
        cudaMemPool_t pool;
        CUDA_TRY(cudaDeviceGetDefaultMemPool(&pool, dev));
        uint64_t keep = UINT64_MAX;
        CUDA_TRY(cudaMemPoolSetAttribute(pool, cudaMemPoolAttrReleaseThreshold, &keep));
        pool_kept[dev] = true;
    }
    return OEQB_OK;
}

// dW = sum over the batch, on the tensor cores: the sums of every tile of 64 items are one row of a partials matrix (the
// tensor cores' accumulation truncates, so it is kept that short), oeq_generic_dw_reduce adds the rows in order.
int tc_backward_dw(Entry* e, const void* x, const void* y, const void* g, void* dW, long long batch, int accum, cudaStream_t st) {
    int rc;
    const Desc& d = e->d;
    TcDwParams p{x, y, g, nullptr, batch, 0, 0, nullptr};
    if ((rc = status_word(&p.status))) return rc;
    Program *prog, *gen;
    if ((rc = get_program(e, FAM_UVW_TC_DW, &prog))) return rc;
    if ((rc = get_program(e, FAM_GENERIC, &gen))) return rc;
    cudaKernel_t k, kr;
    const size_t smem = d.tc_dw_smem;
    if ((rc = get_kernel(prog, "oeq_uvw_tc_backward_dw", smem, &k))) return rc;
    if ((rc = get_kernel(gen, "oeq_generic_dw_reduce", 0, &kr))) return rc;
    long long tiles = (batch + 63) / 64, grid = sm_count();
    if (grid > tiles) grid = tiles;
    if ((rc = keep_pool_memory())) return rc;
    void* part = nullptr;
    CUDA_TRY(cudaMallocAsync(&part, (size_t)tiles * d.wn * sizeof(float), st));   // one row per tile of 64 items
    p.part = part;
    // the accumulators of 16 groups fill the tensor memory: more groups take more launches (each writes its groups' part
    // of every tile's row)
    const int ngrp = d.tc_ngrp;
    for (int g0 = 0; g0 < ngrp && !rc; g0 += 16) {
        p.grp_begin = g0;
        p.grp_end = std::min(ngrp, g0 + 16);
        void* args[] = {&p};
        rc = launch(k, (unsigned)grid, 16 * 32 + 32, smem, args, st);   // TC_THREADS
    }
    if (!rc) {
        void* rargs[] = {&part, &tiles, &dW, &accum};
        rc = launch(kr, (unsigned)((d.wn + 31) / 32), 256, 0, rargs, st);
    }
    cudaFreeAsync(part, st);
    return rc;
}

// 'uvw' backward on the tensor cores; mask selects the outputs (1 dx, 2 dy, 4 dW).  dx is contracted with y_dx, dW with
// y_dw (they differ in the second-order pass); accum adds to the outputs.
int tc_backward(Entry* e, int mask, const void* x, const void* y_dx, const void* y_dw, const void* W, const void* g, void* dx,
                void* dy, void* dW, long long batch, int accum, cudaStream_t st) {
    if (mask & 1) {   // dx: the forward kernel on the transposed tables, with g in the place of x
        TcParams t{g, y_dx, W, dx, nullptr, batch, accum, nullptr};
        if (int rc = tc_forward(e, t, st, 1)) return rc;
    }
    if (mask & 2) {   // dy: g' = g W^T on the tensor cores, folded with x per item
        TcParams t{x, nullptr, W, dy, g, batch, accum, nullptr};
        if (int rc = tc_forward(e, t, st, 2)) return rc;
    }
    if (mask & 4)     // dW: reduction over the batch on the tensor cores, fixed-order sum of the CTAs' rows
        if (int rc = tc_backward_dw(e, x, y_dw, g, dW, batch, accum, st)) return rc;
    return OEQB_OK;
}

// A problem that the specialised kernels serve took a slower route: counted (oeqb_slow_path_count) and, with the log
// option, reported, so that a performance cliff caused by an unaligned buffer or a missing workspace is visible.
std::atomic<long long> g_slow_paths{0};
void note_slow_path(const char* where, const char* why) {
    g_slow_paths.fetch_add(1, std::memory_order_relaxed);
    if (g_log) fprintf(stderr, "[oeq_b200] %s: %s\n", where, why);
}

// Index validation of a convolution call (caller holds g_mutex).  The channel-parallel kernels turn rows / cols /
// transpose_perm straight into addresses of bulk copies, so a bad entry would be a wild access on a shared GPU.  One
// small kernel checks the arrays, the host waits for it and reads the status word, and the call is refused with
// OEQB_EINVAL before any of the main kernels is launched.  The wait makes this a synchronising step, so by default it runs
// once per edge list (identified by its addresses and sizes; option "validate": 0 never, 2 every call) and never while
// the stream is being captured.
struct GraphKey {
    int dev; const void* rows; const void* cols; const void* perm; long long E, N; int sorted;
    bool operator<(const GraphKey& o) const {
        return std::tie(dev, rows, cols, perm, E, N, sorted) < std::tie(o.dev, o.rows, o.cols, o.perm, o.E, o.N, o.sorted);
    }
};
std::set<GraphKey> g_validated;

int validate_graph(const Desc& d, long long N, long long NS, long long E, const void* rows, const void* cols, const void* perm,
                   bool need_sorted, cudaStream_t st, const char* what) {
    if (g_validate <= 0 || E <= 0) return OEQB_OK;
    GraphKey key{0, rows, cols, perm, E, N * 0x100000001LL + NS, need_sorted ? 1 : 0};
    CUDA_TRY(cudaGetDevice(&key.dev));
    if (g_validate == 1 && g_validated.count(key)) return OEQB_OK;
    cudaStreamCaptureStatus cap = cudaStreamCaptureStatusNone;
    if (cudaStreamIsCapturing(st, &cap) != cudaSuccess || cap != cudaStreamCaptureStatusNone) return OEQB_OK;
    int* status = nullptr;
    if (int rc = status_word(&status)) return rc;
    const unsigned grid = (unsigned)((E + 255) / 256 < 2048 ? (E + 255) / 256 : 2048);
    if (d.idx == 3) gprep::validate_edges<int><<<grid, 256, 0, st>>>((const int*)rows, (const int*)cols, (const int*)perm, E, N, NS, need_sorted, status);
    else gprep::validate_edges<long long><<<grid, 256, 0, st>>>((const long long*)rows, (const long long*)cols, (const long long*)perm, E, N, NS, need_sorted, status);
    g_launches.fetch_add(1, std::memory_order_relaxed);
    CUDA_TRY(cudaGetLastError());
    CUDA_TRY(cudaStreamSynchronize(st));
    int dev = key.dev;
    const int code = *(volatile int*)g_status_host[dev];
    if (code == gprep::STATUS_BAD_INDEX) {
        *(volatile int*)g_status_host[dev] = 0;
        return fail(OEQB_EINVAL, "%s: rows must lie in [0, %lld) and cols in [0, %lld)%s%s; nothing was launched", what, N, NS,
                    need_sorted ? ", rows must be sorted (deterministic convolution)" : "",
                    perm ? ", transpose_perm in [0, n_edges)" : "");
    }
    if (g_validated.size() >= 256) g_validated.clear();
    g_validated.insert(key);
    return OEQB_OK;
}

int check_ptrs(std::initializer_list<const void*> ptrs, const char* what) {
    for (const void* p : ptrs)
        if (!p) return fail(OEQB_EINVAL, "%s: null pointer argument", what);
    return OEQB_OK;
}

}  // namespace

// =============================================================================================== C ABI
extern "C" {

const char* oeqb_last_error(void) { return g_err.c_str(); }
const char* oeqb_version(void) { return "oeq_b200 0.1 (sm_100a)"; }
int64_t oeqb_launch_count(void) { return g_launches.load(); }

int oeqb_set_option(const char* name, const char* value) {
    if (!name || !value) return fail(OEQB_EINVAL, "oeqb_set_option: null argument");
    std::lock_guard<std::mutex> lock(g_mutex);
    std::string n = name;
    if (n == "cache_dir") g_cache_dir = value;
    else if (n == "force_generic") g_force_generic = atoi(value) != 0;
    else if (n == "log") g_log = atoi(value) != 0;
    else if (n == "single_group") g_single_group = atoi(value) != 0;
    else if (n == "single_producer") g_single_producer = atoi(value) != 0;
    else if (n == "streams") g_streams = atoi(value);
    else if (n == "streams_forward") g_streams_fwd = atoi(value) != 0;
    else if (n == "validate") g_validate = atoi(value);
    else if (n == "no_tc") g_no_tc = atoi(value) != 0;
    else if (n == "tc_backward") g_tc_backward = atoi(value) & 7;
    else return fail(OEQB_EINVAL, "unknown option '%s'", name);
    return OEQB_OK;
}

int oeqb_query(const void* desc, size_t desc_len, int64_t key, oeqb_kernel_prop* out) {
    if (!out) return fail(OEQB_EINVAL, "oeqb_query: null output");
    std::lock_guard<std::mutex> lock(g_mutex);
    Entry* e;
    int rc = get_entry(desc, desc_len, key, &e);
    if (rc) return rc;
    const Desc& d = e->d;
    memset(out, 0, sizeof *out);
    out->L1_dim = d.dim[0]; out->L2_dim = d.dim[1]; out->L3_dim = d.dim[2]; out->weight_numel = d.wn;
    out->shared_weights = d.shared; out->irrep_dtype = d.dtype; out->weight_dtype = d.dtype; out->idx_dtype = d.idx;
    out->is_conv = d.conv; out->deterministic = d.det; out->kahan = d.kahan; out->is_uvw = d.uvw;
    out->fast_path = (d.fast && !g_force_generic) ? 1 : ((d.tc && !g_force_generic && !g_no_tc) ? 2 : 0);
    return OEQB_OK;
}

int oeqb_emit_source(const void* desc, size_t desc_len, const char* kind, char* buf, size_t cap, size_t* needed) {
    if (!desc || !kind) return fail(OEQB_EINVAL, "oeqb_emit_source: null argument");
    Desc d;
    std::string why;
    if (!parse_desc((const char*)desc, desc_len, d, why)) return fail(OEQB_EPARSE, "descriptor: %s", why.c_str());
    int fam = family_from_name(kind);
    if (fam < 0) return fail(OEQB_EINVAL, "unknown kernel family '%s'", kind);
    std::string src = family_source(d, emit_header(d), fam);
    if (needed) *needed = src.size() + 1;
    if (buf && cap) {
        size_t n = src.size() < cap - 1 ? src.size() : cap - 1;
        memcpy(buf, src.data(), n);
        buf[n] = '\0';
    }
    return OEQB_OK;
}

int oeqb_precompile(const void* desc, size_t desc_len, int64_t key) {
    (void)key;
    if (!desc) return -fail(OEQB_EINVAL, "oeqb_precompile: null descriptor");
    Desc d;
    std::string why;
    if (!parse_desc((const char*)desc, desc_len, d, why)) return -fail(OEQB_EPARSE, "descriptor: %s", why.c_str());
    std::lock_guard<std::mutex> lock(g_mutex);
    const std::string header = emit_header(d);
    int done = 0;
    for (int fam = 0; fam < FAM_COUNT; ++fam) {
        if (fam == FAM_UVW_TC) { if (!d.tc) continue; }
        else if (fam >= FAM_UVW_TC_DX && fam <= FAM_UVW_TC_DW) { if (!d.tc_bwd) continue; }
        else if (fam != FAM_GENERIC && !d.fast) continue;
        if (fam >= FAM_FAST_BWD2_TP && fam <= FAM_FAST_BWD2_ATOMIC && d.fast_S4 < 3) continue;
        if (fam == FAM_FAST_FWD_ATOMIC && d.fast_S3 < 2) continue;
        if ((fam == FAM_FAST_FWD3_TP || fam == FAM_FAST_FWD3_DET) && d.fast_S4 < 3) continue;
        std::string cubin;
        int rc = compile_cubin(family_source(d, header, fam), family_name(fam), cubin);
        if (rc) return -rc;
        ++done;
        if (family_streams(d, fam, true) > 1) {   // the one-stream variant too: it is the fallback
            rc = compile_cubin(family_source(d, header, fam, false), family_name(fam), cubin);
            if (rc) return -rc;
            ++done;
        }
    }
    return done;
}

int oeqb_tp_forward(const void* desc, size_t desc_len, int64_t key, int64_t batch, const void* x, const void* y,
                    const void* W, void* z, void* stream) {
    if (batch < 0) return fail(OEQB_EINVAL, "oeqb_tp_forward: negative batch");
    if (batch == 0) return OEQB_OK;
    if (int rc = check_ptrs({x, y, W, z}, "oeqb_tp_forward")) return rc;
    std::lock_guard<std::mutex> lock(g_mutex);
    Entry* e;
    if (int rc = get_entry(desc, desc_len, key, &e)) return rc;
    if (use_fast(e->d) && aligned16({x, W})) {
        FastParams f{x, y, W, nullptr, z, nullptr, nullptr, nullptr, nullptr, nullptr, nullptr, batch, batch, nullptr};
        return fast_launch(e, 0, f, (cudaStream_t)stream);
    }
    if (e->d.tc && !g_force_generic && !g_no_tc && aligned16({x, z})) {
        TcParams t{x, y, W, z, nullptr, batch, 0, nullptr};
        return tc_forward(e, t, (cudaStream_t)stream);
    }
    FwdParams p{x, y, W, z, nullptr, nullptr, batch, batch, UNIT_ITEM, OUT_STORE};
    return generic_forward(e, p, (cudaStream_t)stream);
}

int oeqb_tp_backward(const void* desc, size_t desc_len, int64_t key, int64_t batch, const void* x, const void* y,
                     const void* W, const void* g, void* dx, void* dy, void* dW, void* stream) {
    if (batch < 0) return fail(OEQB_EINVAL, "oeqb_tp_backward: negative batch");
    if (int rc = check_ptrs({x, y, W, g, dx, dy, dW}, "oeqb_tp_backward")) return rc;
    std::lock_guard<std::mutex> lock(g_mutex);
    Entry* e;
    if (int rc = get_entry(desc, desc_len, key, &e)) return rc;
    cudaStream_t st = (cudaStream_t)stream;
    const Desc& d = e->d;
    if (d.shared) CUDA_TRY(cudaMemsetAsync(dW, 0, d.wn * d.elt(), st));
    if (batch == 0) return OEQB_OK;
    if (use_fast(d) && aligned16({x, W, dx})) {
        FastParams f{x, y, W, g, nullptr, dx, dy, dW, nullptr, nullptr, nullptr, batch, batch, nullptr};
        return fast_launch(e, 3, f, st);
    }
    const int tcb = (d.tc_bwd && !g_force_generic && !g_no_tc && aligned16({x, dx, g})) ? g_tc_backward : 0;
    if (tcb != 7) {
        CUDA_TRY(cudaMemsetAsync(dy, 0, batch * d.dim[1] * d.elt(), st));
        BwdParams p{x, y, y, W, g, dx, dy, dW, nullptr, nullptr, nullptr, batch, batch, UNIT_ITEM, 0};
        if (int rc = generic_backward(e, p, st)) return rc;
    }
    return tc_backward(e, tcb, x, y, y, W, g, dx, dy, dW, batch, 0, st);
}

int oeqb_tp_double_backward(const void* desc, size_t desc_len, int64_t key, int64_t batch, const void* x,
                            const void* y, const void* W, const void* g, const void* x2, const void* y2,
                            const void* W2, void* dx, void* dy, void* dW, void* dg, void* stream) {
    if (batch < 0) return fail(OEQB_EINVAL, "oeqb_tp_double_backward: negative batch");
    if (int rc = check_ptrs({x, y, W, g, x2, y2, W2, dx, dy, dW, dg}, "oeqb_tp_double_backward")) return rc;
    std::lock_guard<std::mutex> lock(g_mutex);
    Entry* e;
    if (int rc = get_entry(desc, desc_len, key, &e)) return rc;
    cudaStream_t st = (cudaStream_t)stream;
    const Desc& d = e->d;
    if (d.shared) CUDA_TRY(cudaMemsetAsync(dW, 0, d.wn * d.elt(), st));
    if (batch == 0) return OEQB_OK;
    int rc;
    if (use_fast(d) && d.fast_S4 >= 3 && aligned16({x, x2, W, W2, dx})) {
        // same decomposition on the channel-parallel kernels: three forward passes (store, add, add) and two
        // second-order backward passes (the second adds); see the general path below for the algebra
        if (d.fast_S4 >= 3 && aligned16({dg})) {   // all three terms of dg in one pass
            FastParams f{x, y, W, nullptr, dg, nullptr, nullptr, nullptr, nullptr, nullptr, nullptr, batch, batch, nullptr};
            f.X2 = x2; f.Y2 = y2; f.W2 = W2;
            if ((rc = fast_launch(e, 0, f, st, nullptr, true))) return rc;
        } else {
            FastParams f{x2, y, W, nullptr, dg, nullptr, nullptr, nullptr, nullptr, nullptr, nullptr, batch, batch, nullptr};
            if ((rc = fast_launch(e, 0, f, st))) return rc;
            f.X = x; f.Y = y2; f.accum = 1;
            if ((rc = fast_launch(e, 0, f, st))) return rc;
            f.Y = y; f.W = W2;
            if ((rc = fast_launch(e, 0, f, st))) return rc;
        }
        FastParams b{x, y, W, g, nullptr, dx, dy, dW, nullptr, nullptr, nullptr, batch, batch, nullptr};
        b.X2 = x2; b.Y2 = y2; b.W2 = W2;   // both second-order backward terms in one pass
        return fast_launch(e, 3, b, st, nullptr, true);
    }
    if (d.tc_bwd && !g_force_generic && !g_no_tc && g_tc_backward == 7 && aligned16({x, x2, dx, dg, g})) {
        // the same five passes on the tensor-core kernels (the second and later ones add to their outputs)
        TcParams t{x2, y, W, dg, nullptr, batch, 0, nullptr};
        if ((rc = tc_forward(e, t, st, 0))) return rc;
        t.x = x; t.y = y2; t.accum = 1;
        if ((rc = tc_forward(e, t, st, 0))) return rc;
        t.y = y; t.W = W2;
        if ((rc = tc_forward(e, t, st, 0))) return rc;
        if ((rc = tc_backward(e, 7, x2, y2, y, W, g, dx, dy, dW, batch, 0, st))) return rc;
        return tc_backward(e, 7, x, y, y2, W2, g, dx, dy, dW, batch, 1, st);
    }
    CUDA_TRY(cudaMemsetAsync(dy, 0, batch * d.dim[1] * d.elt(), st));
    // dg = F(x2, y, W) + F(x, y2, W) + F(x, y, W2): the product is linear in each argument
    FwdParams f{x2, y, W, dg, nullptr, nullptr, batch, batch, UNIT_ITEM, OUT_STORE};
    if ((rc = generic_forward(e, f, st))) return rc;
    f.x = x; f.y = y2; f.out_mode = OUT_ADD;
    if ((rc = generic_forward(e, f, st))) return rc;
    f.y = y; f.W = W2;
    if ((rc = generic_forward(e, f, st))) return rc;
    // (dx, dy, dW) = mixed second derivatives contracted with g
    BwdParams b{x2, y2, y, W, g, dx, dy, dW, nullptr, nullptr, nullptr, batch, batch, UNIT_ITEM, 0};
    if ((rc = generic_backward(e, b, st))) return rc;
    b.x = x; b.y_dx = y; b.y_dw = y2; b.W = W2; b.accum = 1;
    return generic_backward(e, b, st);
}

int64_t oeqb_conv_workspace_bytes(const void* desc, size_t desc_len, int64_t key, int direction, int64_t n_nodes,
                                  int64_t n_edges) {
    if (n_nodes < 0 || n_edges < 0 || direction < 0 || direction > 2)
        return -(int64_t)fail(OEQB_EINVAL, "oeqb_conv_workspace_bytes: bad argument");
    std::lock_guard<std::mutex> lock(g_mutex);
    Entry* e;
    if (int rc = get_entry(desc, desc_len, key, &e)) return -(int64_t)rc;
    const Desc& d = e->d;
    // Deterministic backward on the channel-parallel path: one dX row per edge plus the sender offsets.
    if ((direction == 1 || (direction == 2 && d.fast_S4 >= 3)) && d.conv && d.det && use_fast(d))
        return (int64_t)(round_up((size_t)n_edges * d.dim[0] * d.elt()) + round_up((size_t)(n_nodes + 1) * 8));
    // Unsorted (atomic) convolutions on the channel-parallel path: room to group the edge list by receiver first.
    if (d.conv && !d.det && use_fast(d) && n_edges > 0) return (int64_t)atomic_order_bytes(d, n_nodes, n_edges);
    return 0;
}

static int conv_check(const Desc& d, int64_t n_nodes, int64_t n_edges, const void* perm, const char* what) {
    if (n_nodes < 0 || n_edges < 0) return fail(OEQB_EINVAL, "%s: negative size", what);
    if (!d.conv) return fail(OEQB_EINVAL, "%s: descriptor was not built for a convolution", what);
    if (d.det && n_edges > 0 && !perm) return fail(OEQB_EINVAL, "%s: deterministic mode needs transpose_perm", what);
    return OEQB_OK;
}

static int conv_backward_impl(const void* desc, size_t desc_len, int64_t key, int64_t n_receivers, int64_t n_nodes,
                              int64_t n_edges, const void* X, const void* Y, const void* W, const void* G, void* dX,
                              void* dY, void* dW, const void* rows, const void* cols, const void* transpose_perm,
                              void* workspace, int64_t workspace_bytes, void* stream, bool defer_rows);

int oeqb_conv_forward(const void* desc, size_t desc_len, int64_t key, int64_t n_nodes, int64_t n_edges,
                      const void* X, const void* Y, const void* W, void* Z, const void* rows, const void* cols,
                      const void* transpose_perm, void* workspace, int64_t workspace_bytes, void* stream) {
    return oeqb_conv_forward_rect(desc, desc_len, key, n_nodes, n_nodes, n_edges, X, Y, W, Z, rows, cols, transpose_perm,
                                  workspace, workspace_bytes, stream);
}

int oeqb_conv_forward_rect(const void* desc, size_t desc_len, int64_t key, int64_t n_nodes, int64_t n_senders,
                           int64_t n_edges, const void* X, const void* Y, const void* W, void* Z, const void* rows,
                           const void* cols, const void* transpose_perm, void* workspace, int64_t workspace_bytes,
                           void* stream) {
    if (n_senders < 0) return fail(OEQB_EINVAL, "oeqb_conv_forward_rect: negative size");
    std::lock_guard<std::mutex> lock(g_mutex);
    Entry* e;
    if (int rc = get_entry(desc, desc_len, key, &e)) return rc;
    const Desc& d = e->d;
    if (int rc = conv_check(d, n_nodes, n_edges, transpose_perm, "oeqb_conv_forward")) return rc;
    if (n_nodes == 0) return OEQB_OK;
    if (int rc = check_ptrs({X, Z}, "oeqb_conv_forward")) return rc;
    if (n_edges > 0) if (int rc = check_ptrs({Y, W, rows, cols}, "oeqb_conv_forward")) return rc;
    cudaStream_t st = (cudaStream_t)stream;
    if (int rc = validate_graph(d, n_nodes, n_senders, n_edges, rows, cols, nullptr, d.det != 0, st, "oeqb_conv_forward")) return rc;
    const bool fast = use_fast(d) && n_edges > 0 && aligned16({X, W});
    if (use_fast(d) && n_edges > 0 && !fast) note_slow_path("oeqb_conv_forward", "X or W is not 16-byte aligned: general kernels");
    if (d.det) {
        if (fast) {
            FastParams f{X, Y, W, nullptr, Z, nullptr, nullptr, nullptr, nullptr, rows, cols, n_nodes, n_edges, nullptr};
            return fast_launch(e, 1, f, st);
        }
        FwdParams p{X, Y, W, Z, rows, cols, n_nodes, n_edges, UNIT_SEGMENT, OUT_STORE};
        return generic_forward(e, p, st);
    }
    if (fast) {
        // Group the edges by receiver on the device, then run the sorted-list kernel through that order: each
        // receiver row is summed in registers and written once, instead of one 50 KB read-modify-write per edge.
        const void* order = nullptr;
        const int grc = group_by_receiver(d, n_nodes, n_edges, rows, workspace, workspace_bytes, st, &order);
        if (grc > 0) return grc;
        if (grc == 0) {
            FastParams f{X, Y, W, nullptr, Z, nullptr, nullptr, nullptr, nullptr, rows, cols, n_nodes, n_edges, nullptr};
            f.eorder = order;
            return fast_launch(e, 1, f, st);
        }
        note_slow_path("oeqb_conv_forward", "no workspace for grouping the edges by receiver: per-edge scatter");
    }
    CUDA_TRY(cudaMemsetAsync(Z, 0, n_nodes * d.dim[2] * d.elt(), st));
    if (fast && d.fast_S3 >= 2 && aligned16({Z})) {
        FastParams f{X, Y, W, nullptr, Z, nullptr, nullptr, nullptr, nullptr, rows, cols, n_nodes, n_edges, nullptr};
        return fast_launch(e, 2, f, st);
    }
    FwdParams p{X, Y, W, Z, rows, cols, n_edges, n_edges, UNIT_EDGE, OUT_ATOMIC};
    return generic_forward(e, p, st);
}

int oeqb_conv_backward(const void* desc, size_t desc_len, int64_t key, int64_t n_nodes, int64_t n_edges,
                       const void* X, const void* Y, const void* W, const void* G, void* dX, void* dY, void* dW,
                       const void* rows, const void* cols, const void* transpose_perm, void* workspace,
                       int64_t workspace_bytes, void* stream) {
    return oeqb_conv_backward_rect(desc, desc_len, key, n_nodes, n_nodes, n_edges, X, Y, W, G, dX, dY, dW, rows, cols,
                                   transpose_perm, workspace, workspace_bytes, stream);
}

int oeqb_conv_backward_rect(const void* desc, size_t desc_len, int64_t key, int64_t n_receivers, int64_t n_nodes,
                            int64_t n_edges, const void* X, const void* Y, const void* W, const void* G, void* dX,
                            void* dY, void* dW, const void* rows, const void* cols, const void* transpose_perm,
                            void* workspace, int64_t workspace_bytes, void* stream) {
    return conv_backward_impl(desc, desc_len, key, n_receivers, n_nodes, n_edges, X, Y, W, G, dX, dY, dW, rows, cols,
                              transpose_perm, workspace, workspace_bytes, stream, /*defer_rows=*/false);
}

int oeqb_conv_backward_edges(const void* desc, size_t desc_len, int64_t key, int64_t n_receivers, int64_t n_nodes,
                             int64_t n_edges, const void* X, const void* Y, const void* W, const void* G, void* dY,
                             void* dW, const void* rows, const void* cols, const void* transpose_perm, void* workspace,
                             int64_t workspace_bytes, void* stream) {
    // dX is not touched by this step; a non-null placeholder satisfies the common argument checks
    return conv_backward_impl(desc, desc_len, key, n_receivers, n_nodes, n_edges, X, Y, W, G, workspace, dY, dW, rows, cols,
                              transpose_perm, workspace, workspace_bytes, stream, /*defer_rows=*/true);
}

int oeqb_conv_backward_rows(const void* desc, size_t desc_len, int64_t key, int64_t n_nodes, int64_t n_edges,
                            int64_t row_begin, int64_t row_end, const void* transpose_perm, void* workspace,
                            int64_t workspace_bytes, void* dX, void* stream) {
    if (row_begin < 0 || row_end > n_nodes || row_begin > row_end)
        return fail(OEQB_EINVAL, "oeqb_conv_backward_rows: bad row range [%lld, %lld) of %lld", (long long)row_begin,
                    (long long)row_end, (long long)n_nodes);
    std::lock_guard<std::mutex> lock(g_mutex);
    Entry* e;
    if (int rc = get_entry(desc, desc_len, key, &e)) return rc;
    const Desc& d = e->d;
    if (!(d.conv && d.det && use_fast(d)))
        return fail(OEQB_EUNSUPPORTED, "oeqb_conv_backward_rows: only after oeqb_conv_backward_edges (deterministic "
                                       "convolutions on the channel-parallel kernels)");
    const size_t scratch_bytes = round_up((size_t)n_edges * d.dim[0] * d.elt());
    const size_t need = scratch_bytes + round_up((size_t)(n_nodes + 1) * 8);
    if (!workspace || workspace_bytes < (int64_t)need || !dX || !transpose_perm || !aligned16({workspace, dX}))
        return fail(OEQB_EINVAL, "oeqb_conv_backward_rows: needs the workspace of the matching oeqb_conv_backward_edges call "
                                 "(%zu bytes), dX and transpose_perm", need);
    return fast_scatter_rows(e, workspace, transpose_perm, (char*)workspace + scratch_bytes, row_begin, row_end, dX,
                             (cudaStream_t)stream);
}

static int conv_backward_impl(const void* desc, size_t desc_len, int64_t key, int64_t n_receivers, int64_t n_nodes,
                              int64_t n_edges, const void* X, const void* Y, const void* W, const void* G, void* dX,
                              void* dY, void* dW, const void* rows, const void* cols, const void* transpose_perm,
                              void* workspace, int64_t workspace_bytes, void* stream, bool defer_rows) {
    if (n_receivers < 0) return fail(OEQB_EINVAL, "oeqb_conv_backward_rect: negative size");
    std::lock_guard<std::mutex> lock(g_mutex);
    Entry* e;
    if (int rc = get_entry(desc, desc_len, key, &e)) return rc;
    const Desc& d = e->d;
    if (int rc = conv_check(d, n_nodes, n_edges, transpose_perm, "oeqb_conv_backward")) return rc;
    cudaStream_t st = (cudaStream_t)stream;
    if (d.shared) { if (!dW) return fail(OEQB_EINVAL, "oeqb_conv_backward: null dW"); CUDA_TRY(cudaMemsetAsync(dW, 0, d.wn * d.elt(), st)); }
    if (n_nodes == 0) return OEQB_OK;
    if (int rc = check_ptrs({X, G, dX}, "oeqb_conv_backward")) return rc;
    if (n_edges > 0) {
        if (int rc = check_ptrs({Y, W, dY, dW, rows, cols}, "oeqb_conv_backward")) return rc;
        if (int rc = validate_graph(d, n_receivers, n_nodes, n_edges, rows, cols, d.det ? transpose_perm : nullptr, d.det != 0, st, "oeqb_conv_backward")) return rc;
    }
    const bool fast = use_fast(d) && n_edges > 0 && aligned16({X, W, G, dX, workspace});
    if (use_fast(d) && n_edges > 0 && !fast) note_slow_path("oeqb_conv_backward", "an operand is not 16-byte aligned: general kernels");
    if (d.det && fast) {
        const size_t scratch_bytes = round_up((size_t)n_edges * d.dim[0] * d.elt());
        const size_t need = scratch_bytes + round_up((size_t)(n_nodes + 1) * 8);
        if (!workspace || workspace_bytes < (int64_t)need)
            return fail(OEQB_EINVAL, "oeqb_conv_backward: workspace of %lld bytes is smaller than the %zu required",
                        (long long)workspace_bytes, need);
        void* colptr = (char*)workspace + scratch_bytes;
        FastParams f{X, Y, W, G, nullptr, dX, dY, dW, workspace, rows, cols, n_nodes, n_edges, nullptr};
        if (int rc = fast_launch(e, 4, f, st)) return rc;
        if (defer_rows) return fast_scatter_offsets(e, cols, transpose_perm, n_nodes, n_edges, colptr, st);
        return fast_scatter(e, workspace, cols, transpose_perm, n_nodes, n_edges, colptr, dX, st);
    }
    if (defer_rows)
        return fail(OEQB_EUNSUPPORTED, "oeqb_conv_backward_edges: this problem (or these buffers) is not served by the "
                                       "deterministic channel-parallel kernels; call oeqb_conv_backward");
    if (!d.det && fast) {
        CUDA_TRY(cudaMemsetAsync(dX, 0, n_nodes * d.dim[0] * d.elt(), st));
        FastParams f{X, Y, W, G, nullptr, dX, dY, dW, nullptr, rows, cols, n_nodes, n_edges, nullptr};
        // walked receiver by receiver (grouped on the device), a receiver's gradient row is read once, not once per edge
        const int grc = group_by_receiver(d, n_nodes, n_edges, rows, workspace, workspace_bytes, st, &f.eorder);
        if (grc > 0) return grc;
        if (grc < 0) note_slow_path("oeqb_conv_backward", "no workspace for grouping the edges by receiver");
        return fast_launch(e, 5, f, st);
    }
    if (n_edges > 0) CUDA_TRY(cudaMemsetAsync(dY, 0, n_edges * d.dim[1] * d.elt(), st));
    if (d.det) {
        BwdParams p{X, Y, Y, W, G, dX, dY, dW, rows, cols, transpose_perm, n_nodes, n_edges, UNIT_SEGMENT, 0};
        return generic_backward(e, p, st);
    }
    CUDA_TRY(cudaMemsetAsync(dX, 0, n_nodes * d.dim[0] * d.elt(), st));
    BwdParams p{X, Y, Y, W, G, dX, dY, dW, rows, cols, nullptr, n_edges, n_edges, UNIT_EDGE, 0};
    return generic_backward(e, p, st);
}

int oeqb_conv_double_backward(const void* desc, size_t desc_len, int64_t key, int64_t n_nodes, int64_t n_edges,
                              const void* X, const void* Y, const void* W, const void* G, const void* X2,
                              const void* Y2, const void* W2, void* dX, void* dY, void* dW, void* dG,
                              const void* rows, const void* cols, const void* transpose_perm, void* workspace,
                              int64_t workspace_bytes, void* stream) {
    std::lock_guard<std::mutex> lock(g_mutex);
    Entry* e;
    if (int rc = get_entry(desc, desc_len, key, &e)) return rc;
    const Desc& d = e->d;
    if (int rc = conv_check(d, n_nodes, n_edges, transpose_perm, "oeqb_conv_double_backward")) return rc;
    cudaStream_t st = (cudaStream_t)stream;
    if (d.shared) { if (!dW) return fail(OEQB_EINVAL, "oeqb_conv_double_backward: null dW"); CUDA_TRY(cudaMemsetAsync(dW, 0, d.wn * d.elt(), st)); }
    if (n_nodes == 0) return OEQB_OK;
    if (int rc = check_ptrs({X, G, X2, dX, dG}, "oeqb_conv_double_backward")) return rc;
    if (n_edges > 0) {
        if (int rc = check_ptrs({Y, W, Y2, W2, dY, dW, rows, cols}, "oeqb_conv_double_backward")) return rc;
        if (int rc = validate_graph(d, n_nodes, n_nodes, n_edges, rows, cols, d.det ? transpose_perm : nullptr, d.det != 0, st, "oeqb_conv_double_backward")) return rc;
    }
    int rc;
    if (use_fast(d) && d.fast_S4 >= 3 && (d.det || d.fast_S3 >= 2) && n_edges > 0 && aligned16({X, X2, W, W2, G, dX, dG, workspace})) {
        // channel-parallel kernels: dG from one fused second-order forward pass (three terms), (dX, dY, dW) from one
        // fused second-order backward pass.  An unsorted edge list is grouped by receiver first and then walked through
        // that order by the same kernels as a sorted one; without room for the grouping it takes three accumulating
        // forward passes with a per-edge scatter.
        const int kb = d.det ? 4 : 5;
        void* colptr = nullptr;
        const void* order = nullptr;
        if (d.det) {
            const size_t scratch_bytes = round_up((size_t)n_edges * d.dim[0] * d.elt());
            const size_t need = scratch_bytes + round_up((size_t)(n_nodes + 1) * 8);
            if (!workspace || workspace_bytes < (int64_t)need)
                return fail(OEQB_EINVAL, "oeqb_conv_double_backward: workspace of %lld bytes is smaller than the %zu required",
                            (long long)workspace_bytes, need);
            colptr = (char*)workspace + scratch_bytes;
        } else {
            const int grc = group_by_receiver(d, n_nodes, n_edges, rows, workspace, workspace_bytes, st, &order);
            if (grc > 0) return grc;
            if (grc < 0) note_slow_path("oeqb_conv_double_backward", "no workspace for grouping the edges by receiver");
            CUDA_TRY(cudaMemsetAsync(dX, 0, n_nodes * d.dim[0] * d.elt(), st));
        }
        if (d.det || order) {   // all three terms of dG in one pass over receiver-grouped edges
            FastParams f{X, Y, W, nullptr, dG, nullptr, nullptr, nullptr, nullptr, rows, cols, n_nodes, n_edges, nullptr};
            f.X2 = X2; f.Y2 = Y2; f.W2 = W2; f.eorder = order;
            if ((rc = fast_launch(e, 1, f, st, nullptr, true))) return rc;
        } else {
            CUDA_TRY(cudaMemsetAsync(dG, 0, n_nodes * d.dim[2] * d.elt(), st));
            FastParams f{X2, Y, W, nullptr, dG, nullptr, nullptr, nullptr, nullptr, rows, cols, n_nodes, n_edges, nullptr};
            if ((rc = fast_launch(e, 2, f, st))) return rc;
            f.X = X; f.Y = Y2; f.accum = 1;
            if ((rc = fast_launch(e, 2, f, st))) return rc;
            f.Y = Y; f.W = W2;
            if ((rc = fast_launch(e, 2, f, st))) return rc;
        }
        FastParams b{X, Y, W, G, nullptr, dX, dY, dW, workspace, rows, cols, n_nodes, n_edges, nullptr};
        b.X2 = X2; b.Y2 = Y2; b.W2 = W2; b.eorder = order;   // both second-order backward terms in one pass
        if ((rc = fast_launch(e, kb, b, st, nullptr, true))) return rc;
        if (d.det) return fast_scatter(e, workspace, cols, transpose_perm, n_nodes, n_edges, colptr, dX, st);
        return OEQB_OK;
    }
    if (n_edges > 0) CUDA_TRY(cudaMemsetAsync(dY, 0, n_edges * d.dim[1] * d.elt(), st));
    if (d.det) {
        FwdParams f{X2, Y, W, dG, rows, cols, n_nodes, n_edges, UNIT_SEGMENT, OUT_STORE};
        if ((rc = generic_forward(e, f, st))) return rc;
        f.x = X; f.y = Y2; f.out_mode = OUT_ADD;
        if ((rc = generic_forward(e, f, st))) return rc;
        f.y = Y; f.W = W2;
        if ((rc = generic_forward(e, f, st))) return rc;
        BwdParams b{X2, Y2, Y, W, G, dX, dY, dW, rows, cols, transpose_perm, n_nodes, n_edges, UNIT_SEGMENT, 0};
        if ((rc = generic_backward(e, b, st))) return rc;
        b.x = X; b.y_dx = Y; b.y_dw = Y2; b.W = W2; b.accum = 1;
        return generic_backward(e, b, st);
    }
    CUDA_TRY(cudaMemsetAsync(dG, 0, n_nodes * d.dim[2] * d.elt(), st));
    CUDA_TRY(cudaMemsetAsync(dX, 0, n_nodes * d.dim[0] * d.elt(), st));
    FwdParams f{X2, Y, W, dG, rows, cols, n_edges, n_edges, UNIT_EDGE, OUT_ATOMIC};
    if ((rc = generic_forward(e, f, st))) return rc;
    f.x = X; f.y = Y2;
    if ((rc = generic_forward(e, f, st))) return rc;
    f.y = Y; f.W = W2;
    if ((rc = generic_forward(e, f, st))) return rc;
    BwdParams b{X2, Y2, Y, W, G, dX, dY, dW, rows, cols, nullptr, n_edges, n_edges, UNIT_EDGE, 0};
    if ((rc = generic_backward(e, b, st))) return rc;
    b.x = X; b.y_dx = Y; b.y_dw = Y2; b.W = W2; b.accum = 1;
    return generic_backward(e, b, st);
}


int oeqb_conv_backward_noalloc(const void* desc, size_t desc_len, int64_t key, int64_t n_nodes, int64_t n_edges,
                               const void* X, const void* Y, const void* W, const void* G, void* dX, void* dY, void* dW,
                               const void* rows, const void* cols, const void* transpose_perm, void* stream) {
    std::lock_guard<std::mutex> lock(g_mutex);
    Entry* e;
    if (int rc = get_entry(desc, desc_len, key, &e)) return rc;
    const Desc& d = e->d;
    if (int rc = conv_check(d, n_nodes, n_edges, transpose_perm, "oeqb_conv_backward_noalloc")) return rc;
    if (!(d.det && use_fast(d)))
        return fail(OEQB_EUNSUPPORTED, "oeqb_conv_backward_noalloc: only deterministic convolutions served by the "
                                       "channel-parallel kernels use scratch; call oeqb_conv_backward for this problem");
    if (n_nodes == 0 || n_edges == 0)
        return fail(OEQB_EINVAL, "oeqb_conv_backward_noalloc: empty graph; call oeqb_conv_backward");
    const size_t scratch_bytes = round_up((size_t)n_edges * d.dim[0] * d.elt());
    const size_t colptr_bytes = round_up((size_t)(n_nodes + 1) * 8);
    const size_t need = scratch_bytes + colptr_bytes + kAlign;   // last slot: the kernels' status word
    if (need > (size_t)OEQB_NOALLOC_SCRATCH_BYTES)
        return fail(OEQB_EINVAL, "oeqb_conv_backward_noalloc: this graph needs %zu bytes of scratch (%lld edges x %lld-float "
                                 "rows + %lld sender offsets) but the built-in array holds %zu; use oeqb_conv_backward "
                                 "with a caller-provided workspace",
                    need, (long long)n_edges, (long long)d.dim[0], (long long)n_nodes + 1, (size_t)OEQB_NOALLOC_SCRATCH_BYTES);
    if (int rc = check_ptrs({X, Y, W, G, dX, dY, dW, rows, cols}, "oeqb_conv_backward_noalloc")) return rc;
    if (!aligned16({X, W, G, dX}))
        return fail(OEQB_EINVAL, "oeqb_conv_backward_noalloc: X, W, G and dX must be 16-byte aligned");
    void* base = nullptr;
    if (int rc = noalloc_scratch(&base)) return rc;
    cudaStream_t st = (cudaStream_t)stream;
    void* colptr = (char*)base + scratch_bytes;
    // The kernels' status word sits in the last slot of the array, wherever the graph's rows end, so that
    // oeqb_noalloc_status can find it without knowing the sizes of the call that wrote it.
    int* status = (int*)((char*)base + (size_t)OEQB_NOALLOC_SCRATCH_BYTES - kAlign);
    // The array keeps whatever the previous call left.  Per-edge rows and sender offsets are overwritten in full by
    // the kernels below; only the status word has to start at zero.
    CUDA_TRY(cudaMemsetAsync(status, 0, sizeof(int), st));
    FastParams f{X, Y, W, G, nullptr, dX, dY, dW, base, rows, cols, n_nodes, n_edges, nullptr};
    if (int rc = fast_launch(e, 4, f, st, status)) return rc;
    return fast_scatter(e, base, cols, transpose_perm, n_nodes, n_edges, colptr, dX, st);
}

int oeqb_selftest_bounded_wait(const void* desc, size_t desc_len, int64_t key, void* stream) {
    std::lock_guard<std::mutex> lock(g_mutex);
    Entry* e;
    if (int rc = get_entry(desc, desc_len, key, &e)) return rc;
    if (!use_fast(e->d)) return fail(OEQB_EUNSUPPORTED, "oeqb_selftest_bounded_wait: the descriptor is not served by the channel-parallel kernels");
    int* status = nullptr;
    if (int rc = status_word(&status)) return rc;
    Program* prog;
    if (int rc = get_program(e, FAM_FAST_SCATTER, &prog)) return rc;
    cudaKernel_t k;
    if (int rc = get_kernel(prog, "oeq_selftest_starved_wait", 0, &k)) return rc;
    cudaStream_t st = (cudaStream_t)stream;
    int* left = nullptr;
    CUDA_TRY(cudaMallocAsync((void**)&left, sizeof(int), st));
    CUDA_TRY(cudaMemsetAsync(left, 0, sizeof(int), st));
    void* args[] = {&status, &left};
    int rc = launch(k, 1, 64, 0, args, st);
    int came_back = 0;
    if (!rc) {
        CUDA_TRY(cudaMemcpyAsync(&came_back, left, sizeof(int), cudaMemcpyDeviceToHost, st));
        CUDA_TRY(cudaStreamSynchronize(st));
    }
    cudaFreeAsync(left, st);
    if (rc) return rc;
    // the kernel must have returned (it did: the synchronisation came back), every thread must have left, and the status
    // word must carry the code; reading it clears it
    const int seen = status_word(nullptr);
    if (came_back != 64) return fail(OEQB_EKERNEL, "oeqb_selftest_bounded_wait: %d of 64 threads came back", came_back);
    if (seen != OEQB_EKERNEL) return fail(OEQB_EKERNEL, "oeqb_selftest_bounded_wait: the starved wait did not report through the status word");
    return OEQB_OK;
}

int oeqb_check_status(void) {
    std::lock_guard<std::mutex> lock(g_mutex);
    return status_word(nullptr);
}

int64_t oeqb_slow_path_count(void) { return g_slow_paths.load(); }

int64_t oeqb_graph_workspace_bytes(int64_t n_nodes, int64_t n_edges) {
    if (n_nodes < 0 || n_edges < 0) return -(int64_t)fail(OEQB_EINVAL, "oeqb_graph_workspace_bytes: negative size");
    return (int64_t)gprep::group_workspace_bytes(n_nodes, n_edges);
}

int oeqb_prepare_graph(int idx_dtype, int64_t n_nodes, int64_t n_edges, const void* rows, const void* cols,
                       void* sorted_rows, void* sorted_cols, void* order, void* transpose_perm, void* workspace,
                       int64_t workspace_bytes, void* stream) {
    if (idx_dtype != 3 && idx_dtype != 4) return fail(OEQB_EINVAL, "oeqb_prepare_graph: idx_dtype must be 3 (int32) or 4 (int64)");
    if (n_nodes < 0 || n_edges < 0) return fail(OEQB_EINVAL, "oeqb_prepare_graph: negative size");
    if (n_edges == 0) return OEQB_OK;
    if (n_nodes == 0) return fail(OEQB_EINVAL, "oeqb_prepare_graph: edges without nodes");
    if (int rc = check_ptrs({rows, cols, sorted_rows, sorted_cols, order, transpose_perm, workspace}, "oeqb_prepare_graph")) return rc;
    if (workspace_bytes < (int64_t)gprep::group_workspace_bytes(n_nodes, n_edges) || ((uintptr_t)workspace & 15u))
        return fail(OEQB_EINVAL, "oeqb_prepare_graph: workspace of %lld bytes is smaller than the %zu required (or not 16-byte aligned)",
                    (long long)workspace_bytes, gprep::group_workspace_bytes(n_nodes, n_edges));
    std::lock_guard<std::mutex> lock(g_mutex);
    int* status = nullptr;
    if (int rc = status_word(&status)) return rc;
    cudaStream_t st = (cudaStream_t)stream;
    long long launches = 0;
    bool ok;
    // pass 1: by (row, col) -> order, sorted rows / cols; pass 2: the sorted list by (col, row) -> transpose_perm
    if (idx_dtype == 3) {
        ok = gprep::group_by_key<int>((const int*)rows, (const int*)cols, n_edges, n_nodes, (int*)order, (int*)sorted_rows,
                                      (int*)sorted_cols, workspace, status, st, nullptr, &launches) &&
             gprep::group_by_key<int>((const int*)sorted_cols, (const int*)sorted_rows, n_edges, n_nodes, (int*)transpose_perm,
                                      nullptr, nullptr, workspace, status, st, nullptr, &launches);
    } else {
        ok = gprep::group_by_key<long long>((const long long*)rows, (const long long*)cols, n_edges, n_nodes, (long long*)order,
                                            (long long*)sorted_rows, (long long*)sorted_cols, workspace, status, st, nullptr, &launches) &&
             gprep::group_by_key<long long>((const long long*)sorted_cols, (const long long*)sorted_rows, n_edges, n_nodes,
                                            (long long*)transpose_perm, nullptr, nullptr, workspace, status, st, nullptr, &launches);
    }
    g_launches.fetch_add(launches, std::memory_order_relaxed);
    if (!ok) return fail(OEQB_ECUDA, "oeqb_prepare_graph: kernel launch failed: %s", cudaGetErrorString(cudaGetLastError()));
    return OEQB_OK;
}

namespace {
int plan_bounds(const char* who, int32_t world, const int64_t* bounds, int64_t n_nodes, pplan::Bounds* B) {
    if (world < 1 || world > pplan::MAX_WORLD) return fail(OEQB_EINVAL, "%s: world must be 1 ... %d", who, pplan::MAX_WORLD);
    B->world = world;
    for (int q = 0; q <= world; ++q) {
        B->b[q] = bounds ? bounds[q] : (q == 0 ? 0 : n_nodes);
        if (B->b[q] < 0 || B->b[q] > n_nodes || (q > 0 && B->b[q] < B->b[q - 1])) return fail(OEQB_EINVAL, "%s: bounds must ascend within [0, n_nodes]", who);
    }
    return OEQB_OK;
}
}  // namespace

int64_t oeqb_plan_workspace_bytes(int64_t n_nodes, int64_t n_edges, int64_t n_receivers, int64_t n_owned, int32_t world) {
    if (n_nodes < 0 || n_edges < 0 || n_receivers < 0 || n_owned < 0 || world < 1) return -(int64_t)fail(OEQB_EINVAL, "oeqb_plan_workspace_bytes: bad argument");
    return (int64_t)pplan::layout(n_nodes, n_edges, n_receivers, n_owned, world).total;
}

int oeqb_plan_count(int64_t n_nodes, int64_t n_edges, const void* rows, const void* cols, int64_t recv_begin, int64_t recv_end,
                    int64_t own_begin, int64_t own_end, int32_t world, int32_t rank, const int64_t* bounds, void* workspace,
                    int64_t workspace_bytes, int64_t* counts, void* stream) {
    pplan::Bounds B;
    if (int rc = plan_bounds("oeqb_plan_count", world, bounds, n_nodes, &B)) return rc;
    if (n_nodes < 0 || n_edges < 0 || recv_begin < 0 || recv_end < recv_begin || recv_end > n_nodes || own_begin < 0 || own_end < own_begin ||
        own_end > n_nodes || rank < 0 || rank >= world)
        return fail(OEQB_EINVAL, "oeqb_plan_count: bad range");
    if (int rc = check_ptrs({workspace, counts}, "oeqb_plan_count")) return rc;
    if (n_edges > 0) if (int rc = check_ptrs({rows, cols}, "oeqb_plan_count")) return rc;
    const size_t need = pplan::layout(n_nodes, n_edges, recv_end - recv_begin, own_end - own_begin, world).total;
    if (workspace_bytes < (int64_t)need || ((uintptr_t)workspace & 15u))
        return fail(OEQB_EINVAL, "oeqb_plan_count: workspace of %lld bytes is smaller than the %zu required (or not 16-byte aligned)",
                    (long long)workspace_bytes, need);
    long long launches = 0;
    const bool ok = pplan::count((const long long*)rows, (const long long*)cols, n_nodes, n_edges, recv_begin, recv_end, own_begin, own_end, B,
                                 rank, workspace, (long long*)counts, (cudaStream_t)stream, &launches);
    g_launches.fetch_add(launches, std::memory_order_relaxed);
    if (!ok) return fail(OEQB_ECUDA, "oeqb_plan_count: %s", cudaGetErrorString(cudaGetLastError()));
    return OEQB_OK;
}

int oeqb_plan_fill(int64_t n_nodes, int64_t n_edges, const void* rows, const void* cols, int64_t recv_begin, int64_t recv_end,
                   int64_t own_begin, int64_t own_end, int32_t world, const int64_t* bounds, int64_t e0, int64_t e1, int64_t n_halo,
                   void* workspace, int64_t workspace_bytes, void* halo_ids, void* send_ids, void* rows_local, void* cols_local,
                   void* perm_local, void* stream) {
    pplan::Bounds B;
    if (int rc = plan_bounds("oeqb_plan_fill", world, bounds, n_nodes, &B)) return rc;
    if (e0 < 0 || e1 < e0 || e1 > n_edges || n_halo < 0 || n_halo > n_nodes) return fail(OEQB_EINVAL, "oeqb_plan_fill: bad sizes");
    if (int rc = check_ptrs({workspace}, "oeqb_plan_fill")) return rc;
    if (e1 > e0) if (int rc = check_ptrs({rows, cols, rows_local, cols_local, perm_local}, "oeqb_plan_fill")) return rc;
    const size_t need = pplan::layout(n_nodes, n_edges, recv_end - recv_begin, own_end - own_begin, world).total;
    if (workspace_bytes < (int64_t)need) return fail(OEQB_EINVAL, "oeqb_plan_fill: workspace too small");
    std::lock_guard<std::mutex> lock(g_mutex);
    int* status = nullptr;
    if (int rc = status_word(&status)) return rc;
    long long launches = 0;
    const bool ok = pplan::fill((const long long*)rows, (const long long*)cols, n_nodes, n_edges, recv_begin, recv_end, own_begin, own_end, B, e0,
                                e1, n_halo, workspace, (long long*)halo_ids, (long long*)send_ids, (long long*)rows_local,
                                (long long*)cols_local, (long long*)perm_local, status, (cudaStream_t)stream, &launches);
    g_launches.fetch_add(launches, std::memory_order_relaxed);
    if (!ok) return fail(OEQB_ECUDA, "oeqb_plan_fill: %s", cudaGetErrorString(cudaGetLastError()));
    return OEQB_OK;
}

int oeqb_group_mm(int dtype, int ragged_inner, int64_t num_groups, int64_t num_features, int64_t M, int64_t K,
                  const int64_t* ragged_counts, const void* A, const void* B, void* C, void* stream) {
    if (dtype != 1 && dtype != 2) return fail(OEQB_EINVAL, "oeqb_group_mm: dtype must be 1 (float32) or 2 (float64)");
    if (ragged_inner < 0 || ragged_inner > 2) return fail(OEQB_EINVAL, "oeqb_group_mm: ragged_inner must be 0, 1 or 2");
    if (num_groups < 0 || num_features < 0 || M < 0 || K < 0) return fail(OEQB_EINVAL, "oeqb_group_mm: negative size");
    if (num_groups > gmm::MAX_GROUPS) return fail(OEQB_EUNSUPPORTED, "oeqb_group_mm: at most %d groups", gmm::MAX_GROUPS);
    if (K > 64) return fail(OEQB_EUNSUPPORTED, "oeqb_group_mm: K = %lld exceeds 64", (long long)K);
    if (num_features > 65535) return fail(OEQB_EUNSUPPORTED, "oeqb_group_mm: more than 65535 feature channels");
    if (num_groups == 0 || num_features == 0 || (M == 0 && ragged_inner != 2)) return OEQB_OK;
    if (!ragged_counts) return fail(OEQB_EINVAL, "oeqb_group_mm: null ragged_counts");
    gmm::Offsets offs;
    offs.n_groups = (int)num_groups;
    offs.off[0] = 0;
    for (int64_t g = 0; g < num_groups; ++g) {
        if (ragged_counts[g] < 0) return fail(OEQB_EINVAL, "oeqb_group_mm: negative group size");
        offs.off[g + 1] = offs.off[g] + ragged_counts[g];
    }
    const long long n_nodes = offs.off[num_groups];
    cudaStream_t st = (cudaStream_t)stream;
    const size_t elt = dtype == 2 ? 8 : 4;
    if (ragged_inner == 1) {
        // groups without nodes keep zeros; the kernel writes every row of a non-empty group
        if (int rc = check_ptrs({C}, "oeqb_group_mm")) return rc;
        if (K == 0) return OEQB_OK;
    }
    if (n_nodes == 0) {
        if (ragged_inner == 1) CUDA_TRY(cudaMemsetAsync(C, 0, (size_t)num_groups * num_features * M * K * elt, st));
        return OEQB_OK;
    }
    if (int rc = check_ptrs({A, B, C}, "oeqb_group_mm")) return rc;
    if (ragged_inner == 2) {
        if (K == 0) return OEQB_OK;
        if (M == 0) { CUDA_TRY(cudaMemsetAsync(C, 0, (size_t)n_nodes * num_features * K * elt, st)); return OEQB_OK; }
    }
    if (K == 0) { CUDA_TRY(cudaMemsetAsync(C, 0, (size_t)n_nodes * num_features * M * elt, st)); return OEQB_OK; }
    cudaError_t ce = dtype == 2 ? gmm::dispatch<double>(ragged_inner, offs, n_nodes, num_features, (int)M, (int)K, A, B, C, st)
                                : gmm::dispatch<float>(ragged_inner, offs, n_nodes, num_features, (int)M, (int)K, A, B, C, st);
    if (ce != cudaSuccess) return fail(OEQB_ECUDA, "oeqb_group_mm: kernel launch failed: %s", cudaGetErrorString(ce));
    g_launches.fetch_add(1, std::memory_order_relaxed);
    return OEQB_OK;
}

int oeqb_noalloc_status(void) {
    std::lock_guard<std::mutex> lock(g_mutex);
    void* base = nullptr;
    if (int rc = noalloc_scratch(&base)) return rc;
    int code = 0;
    // 4 bytes out of the built-in array into a stack variable: a copy, not an allocation
    CUDA_TRY(cudaMemcpy(&code, (char*)base + (size_t)OEQB_NOALLOC_SCRATCH_BYTES - kAlign, sizeof(int), cudaMemcpyDeviceToHost));
    if (code != 0)
        return fail(OEQB_EKERNEL, "oeqb_conv_backward_noalloc: a kernel of the last call on this device gave up a bounded "
                                  "wait (code %d); its outputs are invalid", code);
    return OEQB_OK;
}

}  // extern "C"

// General tensor-product / convolution kernels: correct for every supported problem (uvu and uvw, any
// multiplicities and degrees, fp32/fp64, shared or per-item weights, both layouts).  One warp owns one
// "unit" at a time and keeps the unit's output in registers, so a unit is written exactly once and the
// summation order inside it is a pure function of the inputs (no atomics unless the caller asks).
//
//   unit = batch item            (TensorProduct)
//   unit = edge                  (convolution, atomic scatter)
//   unit = receiver / sender     (deterministic convolution: all edges of one node, in list order)
//
// Math (reference kernels: templates/loop_unroll_tp.cuh:4-99 forward, :101-313 backward):
//   uvu  z[u,k] += W[u,v] * sum_ij C[ijk] x[u,i] y[v,j]
//   uvw  z[w,k] += sum_{u,v} W[u,v,w] * sum_ij C[ijk] x[u,i] y[v,j]
#pragma once

#define OEQ_UNIT_ITEM 0
#define OEQ_UNIT_EDGE 1
#define OEQ_UNIT_SEGMENT 2

struct FwdParams {
    const T* x; const T* y; const T* W; T* z;
    const IDX* rows; const IDX* cols;
    long long n_units; long long n_edges;
    int unit_mode; int out_mode;
};

template <int N>
OEQ_DEV void accumulate(T (&acc)[N], T (&comp)[N], const T (&msg)[N]) {
#pragma unroll
    for (int k = 0; k < N; ++k) {
#if OEQ_KAHAN
        const T yk = msg[k] - comp[k];
        const T tk = acc[k] + yk;
        comp[k] = (tk - acc[k]) - yk;
        acc[k] = tk;
#else
        acc[k] += msg[k];
#endif
    }
}

extern "C" __global__ void __launch_bounds__(128) oeq_generic_forward(const FwdParams p) {
    const int lane = threadIdx.x & 31;
    const long long warp0 = (blockIdx.x * (long long)blockDim.x + threadIdx.x) >> 5;
    const long long nwarps = (gridDim.x * (long long)blockDim.x) >> 5;
    for (long long unit = warp0; unit < p.n_units; unit += nwarps) {
        long long e_lo = unit, e_hi = unit + 1, out_row = unit;
        if (p.unit_mode == OEQ_UNIT_EDGE) {
            out_row = (long long)p.rows[unit];
        } else if (p.unit_mode == OEQ_UNIT_SEGMENT) {
            e_lo = lower_bound_ll(p.n_edges, unit, [&](long long k) { return p.rows[k]; });
            e_hi = lower_bound_ll(p.n_edges, unit + 1, [&](long long k) { return p.rows[k]; });
        }
        T* zrow = p.z + out_row * L3_DIM;
        static_for<0, NB3>([&](auto oc) {
            constexpr int O = decltype(oc)::value;
            using B3 = Blk3<O>;
            constexpr int MULPAD3 = (B3::MUL + 31) & ~31;   // every lane walks the loop: the 'uvw' branch shuffles
            for (int c = lane; c < MULPAD3; c += 32) {  // c: channel u (uvu) or w (uvw) of the output block
                const bool live = c < B3::MUL;
                T acc[B3::D], comp[B3::D];
#pragma unroll
                for (int k = 0; k < B3::D; ++k) { acc[k] = T(0); comp[k] = T(0); }
                for (long long e = e_lo; e < e_hi; ++e) {
                    const long long xr = (p.unit_mode == OEQ_UNIT_ITEM) ? e : (long long)p.cols[e];
                    const T* xrow = p.x + xr * L1_DIM;
                    const T* yrow = p.y + e * L2_DIM;
                    const T* wrow = OEQ_SHARED_W ? p.W : p.W + e * WN;
                    static_for<0, NINS>([&](auto ic) {
                        using In = Ins<decltype(ic)::value>;
                        if constexpr (In::O == O) {
                            using B1 = Blk1<In::A>;
                            using B2 = Blk2<In::B>;
                            T msg[In::D3];
#pragma unroll
                            for (int k = 0; k < In::D3; ++k) msg[k] = T(0);
#if !OEQ_UVW
                            T xv[In::D1];
#pragma unroll
                            for (int i = 0; i < In::D1; ++i) xv[i] = live ? xrow[feat_idx<B1::OFF, B1::MUL, B1::D>(c, i)] : T(0);
                            for (int v = 0; v < In::V; ++v) {
                                T yv[In::D2], t[In::D3];
#pragma unroll
                                for (int j = 0; j < In::D2; ++j) yv[j] = yrow[feat_idx<B2::OFF, B2::MUL, B2::D>(v, j)];
#pragma unroll
                                for (int k = 0; k < In::D3; ++k) t[k] = T(0);
                                In::fwd(xv, yv, t);
                                const T w = live ? wrow[widx_uvu<In::U, In::V>(In::WOFF, c, v)] : T(0);
#pragma unroll
                                for (int k = 0; k < In::D3; ++k) msg[k] += w * t[k];
                            }
#else
                            // T[u][k] = sum_{i,j} C x[u,i] y[j] does not depend on the output channel: lane l computes it for
                            // channel u0 + l once, and the u -> w contraction takes it from there by shuffles
                            for (int u0 = 0; u0 < In::U; u0 += 32) {
                                const int uo = u0 + lane;
                                const int ulen = (In::U - u0) < 32 ? (In::U - u0) : 32;
                                T xv[In::D1];
#pragma unroll
                                for (int i = 0; i < In::D1; ++i)
                                    xv[i] = (uo < In::U) ? xrow[feat_idx<B1::OFF, B1::MUL, B1::D>(uo, i)] : T(0);
                                for (int v = 0; v < In::V; ++v) {
                                    T yv[In::D2], t[In::D3];
#pragma unroll
                                    for (int j = 0; j < In::D2; ++j) yv[j] = yrow[feat_idx<B2::OFF, B2::MUL, B2::D>(v, j)];
#pragma unroll
                                    for (int k = 0; k < In::D3; ++k) t[k] = T(0);
                                    In::fwd(xv, yv, t);
                                    for (int ul = 0; ul < ulen; ++ul) {
                                        const T w = live ? wrow[widx_uvw<In::U, In::V, In::WN_>(In::WOFF, u0 + ul, v, c)] : T(0);
#pragma unroll
                                        for (int k = 0; k < In::D3; ++k) msg[k] += w * __shfl_sync(0xffffffffu, t[k], ul);
                                    }
                                }
                            }
#endif
                            accumulate(acc, comp, msg);
                        }
                    });
                }
                if (live) {
#pragma unroll
                    for (int k = 0; k < B3::D; ++k)
                        emit_out(&zrow[feat_idx<B3::OFF, B3::MUL, B3::D>(c, k)], acc[k], p.out_mode);
                }
            }
        });
    }
}

// Backward.  The operand roles are split so that the same kernel serves the second-order pass:
//   dx uses (y_dx, W, g);  dy uses (x, W, g);  dW uses (x, y_dw, g).
// A plain backward passes y_dx == y_dw == y.
struct BwdParams {
    const T* x; const T* y_dx; const T* y_dw; const T* W; const T* g;
    T* dx; T* dy; T* dW;
    const IDX* rows; const IDX* cols; const IDX* perm;
    long long n_units; long long n_edges;
    int unit_mode; int accum;
    T* dW_part;   // shared weights, path-major kernel: [chunks][WN] partial sums, reduced in chunk order afterwards
};

extern "C" __global__ void __launch_bounds__(128) oeq_generic_backward(const BwdParams p) {
    const int lane = threadIdx.x & 31;
    const long long warp0 = (blockIdx.x * (long long)blockDim.x + threadIdx.x) >> 5;
    const long long nwarps = (gridDim.x * (long long)blockDim.x) >> 5;
    const int dx_mode = (p.unit_mode == OEQ_UNIT_EDGE) ? OEQ_OUT_ATOMIC : (p.accum ? OEQ_OUT_ADD : OEQ_OUT_STORE);
    const int dw_mode = OEQ_SHARED_W ? OEQ_OUT_ATOMIC : (p.accum ? OEQ_OUT_ADD : OEQ_OUT_STORE);
    for (long long unit = warp0; unit < p.n_units; unit += nwarps) {
        long long k_lo = unit, k_hi = unit + 1, x_row = unit;
        if (p.unit_mode == OEQ_UNIT_EDGE) {
            x_row = (long long)p.cols[unit];
        } else if (p.unit_mode == OEQ_UNIT_SEGMENT) {
            // sender `unit`: its edges are contiguous in the column-major order that `perm` enumerates
            k_lo = lower_bound_ll(p.n_edges, unit, [&](long long k) { return p.cols[p.perm[k]]; });
            k_hi = lower_bound_ll(p.n_edges, unit + 1, [&](long long k) { return p.cols[p.perm[k]]; });
        }
        const T* xrow = p.x + x_row * L1_DIM;
        T* dxrow = p.dx + x_row * L1_DIM;
        static_for<0, NB1>([&](auto ac) {
            constexpr int A = decltype(ac)::value;
            using B1 = Blk1<A>;
            constexpr int MULPAD = (B1::MUL + 31) & ~31;
            for (int c = lane; c < MULPAD; c += 32) {  // c: channel u of the in1 block
                const bool active = c < B1::MUL;
                T dxacc[B1::D], xv[B1::D];
#pragma unroll
                for (int i = 0; i < B1::D; ++i) {
                    dxacc[i] = T(0);
                    xv[i] = active ? xrow[feat_idx<B1::OFF, B1::MUL, B1::D>(c, i)] : T(0);
                }
                for (long long kk = k_lo; kk < k_hi; ++kk) {
                    const long long e = (p.unit_mode == OEQ_UNIT_SEGMENT) ? (long long)p.perm[kk] : kk;
                    const long long g_row = (p.unit_mode == OEQ_UNIT_ITEM) ? e : (long long)p.rows[e];
                    const T* grow = p.g + g_row * L3_DIM;
                    const T* ydx = p.y_dx + e * L2_DIM;
                    const T* ydw = p.y_dw + e * L2_DIM;
                    const T* wrow = OEQ_SHARED_W ? p.W : p.W + e * WN;
                    T* dwrow = OEQ_SHARED_W ? p.dW : p.dW + e * WN;
                    T* dyrow = p.dy + e * L2_DIM;
                    static_for<0, NINS>([&](auto ic) {
                        using In = Ins<decltype(ic)::value>;
                        if constexpr (In::A == A) {
                            using B2 = Blk2<In::B>;
                            using B3 = Blk3<In::O>;
#if !OEQ_UVW
                            T gv[In::D3];
#pragma unroll
                            for (int k = 0; k < In::D3; ++k)
                                gv[k] = active ? grow[feat_idx<B3::OFF, B3::MUL, B3::D>(c, k)] : T(0);
#endif
                            for (int v = 0; v < In::V; ++v) {
                                T y1[In::D2], y2[In::D2], gp[In::D3], dyp[In::D2], t[In::D3];
#pragma unroll
                                for (int j = 0; j < In::D2; ++j) {
                                    y1[j] = ydx[feat_idx<B2::OFF, B2::MUL, B2::D>(v, j)];
                                    y2[j] = ydw[feat_idx<B2::OFF, B2::MUL, B2::D>(v, j)];
                                    dyp[j] = T(0);
                                }
#pragma unroll
                                for (int k = 0; k < In::D3; ++k) t[k] = T(0);
                                In::fwd(xv, y2, t);
#if !OEQ_UVW
                                const int wi = widx_uvu<In::U, In::V>(In::WOFF, active ? c : 0, v);
                                const T w = active ? wrow[wi] : T(0);
                                T dw = T(0);
#pragma unroll
                                for (int k = 0; k < In::D3; ++k) { gp[k] = w * gv[k]; dw += t[k] * gv[k]; }
                                if (active) emit_out(&dwrow[wi], dw, dw_mode);
#else
#pragma unroll
                                for (int k = 0; k < In::D3; ++k) gp[k] = T(0);
                                for (int w = 0; w < In::WN_; ++w) {
                                    const int wi = widx_uvw<In::U, In::V, In::WN_>(In::WOFF, active ? c : 0, v, w);
                                    const T ww = active ? wrow[wi] : T(0);
                                    T dw = T(0);
#pragma unroll
                                    for (int k = 0; k < In::D3; ++k) {
                                        const T gk = grow[feat_idx<B3::OFF, B3::MUL, B3::D>(w, k)];
                                        gp[k] += ww * gk;
                                        dw += t[k] * gk;
                                    }
                                    if (active) emit_out(&dwrow[wi], dw, dw_mode);
                                }
#endif
                                In::dx(y1, gp, dxacc);
                                In::dy(xv, gp, dyp);
#pragma unroll
                                for (int j = 0; j < In::D2; ++j) {
                                    const T s = warp_sum(dyp[j]);
                                    if (lane == 0) dyrow[feat_idx<B2::OFF, B2::MUL, B2::D>(v, j)] += s;
                                }
                            }
                        }
                    });
                }
                if (active) {
#pragma unroll
                    for (int i = 0; i < B1::D; ++i)
                        emit_out(&dxrow[feat_idx<B1::OFF, B1::MUL, B1::D>(c, i)], dxacc[i], dx_mode);
                }
            }
        });
    }
}

#if OEQ_SHARED_W
// Backward for shared weights, path-major: a warp takes a chunk of consecutive items (or edges) and, for one
// (instruction, v, tile of 32 w) at a time, runs over the chunk keeping that tile of dW in registers; only the chunk's
// sums are added to global dW (one atomic per weight and chunk instead of one per weight and item, which is what the
// reference does: templates/loop_unroll_tp.cuh:258-259).  With p.dW_part the chunk's sums are not added atomically but
// stored as row `chunk` of a partials matrix that oeq_generic_dw_reduce sums in chunk order: dW is then bitwise
// reproducible, whatever the grid.  dX and dY are added to per item, so the caller zeroes them.
// Modes: OEQ_UNIT_ITEM (tensor product) and OEQ_UNIT_EDGE (atomic convolution).
constexpr int OEQ_WTILE = 32;

extern "C" __global__ void __launch_bounds__(128) oeq_generic_backward_shared(const BwdParams p, const int chunk) {
    const int lane = threadIdx.x & 31;
    const long long warp0 = (blockIdx.x * (long long)blockDim.x + threadIdx.x) >> 5;
    const long long nwarps = (gridDim.x * (long long)blockDim.x) >> 5;
    const bool edge_mode = p.unit_mode == OEQ_UNIT_EDGE;
    const long long nchunks = (p.n_edges + chunk - 1) / chunk;
    for (long long unit = warp0; unit < nchunks; unit += nwarps) {
        const long long e_lo = unit * chunk, e_hi = (e_lo + chunk < p.n_edges) ? e_lo + chunk : p.n_edges;
        static_for<0, NINS>([&](auto ic) {
            using In = Ins<decltype(ic)::value>;
            using B1 = Blk1<In::A>;
            using B2 = Blk2<In::B>;
            using B3 = Blk3<In::O>;
            constexpr int MULPAD = (B1::MUL + 31) & ~31;
            for (int c = lane; c < MULPAD; c += 32) {   // c: channel u of the in1 block
                const bool active = c < B1::MUL;
                for (int v = 0; v < In::V; ++v) {
#if !OEQ_UVW
                    const int wi = widx_uvu<In::U, In::V>(In::WOFF, active ? c : 0, v);
                    const T w = active ? p.W[wi] : T(0);
                    T dwacc = T(0);
#else
                    for (int w0 = 0; w0 < In::WN_; w0 += OEQ_WTILE) {
                    T wreg[OEQ_WTILE], dwacc[OEQ_WTILE];
#pragma unroll
                    for (int ww = 0; ww < OEQ_WTILE; ++ww) {
                        const bool in = active && (w0 + ww < In::WN_);
                        wreg[ww] = in ? p.W[widx_uvw<In::U, In::V, In::WN_>(In::WOFF, c, v, w0 + ww)] : T(0);
                        dwacc[ww] = T(0);
                    }
#endif
                    for (long long e = e_lo; e < e_hi; ++e) {
                        const long long x_row = edge_mode ? (long long)p.cols[e] : e;
                        const long long g_row = edge_mode ? (long long)p.rows[e] : e;
                        const T* xrow = p.x + x_row * L1_DIM;
                        const T* grow = p.g + g_row * L3_DIM;
                        T xv[In::D1], y1[In::D2], y2[In::D2], gp[In::D3], t[In::D3], dxp[In::D1], dyp[In::D2];
#pragma unroll
                        for (int i = 0; i < In::D1; ++i) {
                            xv[i] = active ? xrow[feat_idx<B1::OFF, B1::MUL, B1::D>(c, i)] : T(0);
                            dxp[i] = T(0);
                        }
#pragma unroll
                        for (int j = 0; j < In::D2; ++j) {
                            y1[j] = p.y_dx[e * L2_DIM + feat_idx<B2::OFF, B2::MUL, B2::D>(v, j)];
                            y2[j] = p.y_dw[e * L2_DIM + feat_idx<B2::OFF, B2::MUL, B2::D>(v, j)];
                            dyp[j] = T(0);
                        }
#pragma unroll
                        for (int k = 0; k < In::D3; ++k) t[k] = T(0);
                        In::fwd(xv, y2, t);
#if !OEQ_UVW
#pragma unroll
                        for (int k = 0; k < In::D3; ++k) {
                            const T gk = active ? grow[feat_idx<B3::OFF, B3::MUL, B3::D>(c, k)] : T(0);
                            gp[k] = w * gk;
                            dwacc += t[k] * gk;
                        }
#else
#pragma unroll
                        for (int k = 0; k < In::D3; ++k) gp[k] = T(0);
#pragma unroll
                        for (int ww = 0; ww < OEQ_WTILE; ++ww) {
                            if (w0 + ww < In::WN_) {
#pragma unroll
                                for (int k = 0; k < In::D3; ++k) {
                                    const T gk = grow[feat_idx<B3::OFF, B3::MUL, B3::D>(w0 + ww, k)];
                                    gp[k] += wreg[ww] * gk;
                                    dwacc[ww] += t[k] * gk;
                                }
                            }
                        }
#endif
                        In::dx(y1, gp, dxp);
                        In::dy(xv, gp, dyp);
                        if (active) {
                            T* dxrow = p.dx + x_row * L1_DIM;
#pragma unroll
                            for (int i = 0; i < In::D1; ++i)
                                emit_out(&dxrow[feat_idx<B1::OFF, B1::MUL, B1::D>(c, i)], dxp[i], edge_mode ? OEQ_OUT_ATOMIC : OEQ_OUT_ADD);
                        }
#pragma unroll
                        for (int j = 0; j < In::D2; ++j) {
                            const T s = warp_sum(dyp[j]);
                            if (lane == 0) p.dy[e * L2_DIM + feat_idx<B2::OFF, B2::MUL, B2::D>(v, j)] += s;
                        }
                    }
                    T* part = p.dW_part ? p.dW_part + unit * (long long)WN : nullptr;
#if !OEQ_UVW
                    if (active) { if (part) part[wi] = dwacc; else atomicAdd(&p.dW[wi], dwacc); }
#else
                    if (active) {
#pragma unroll
                        for (int ww = 0; ww < OEQ_WTILE; ++ww)
                            if (w0 + ww < In::WN_) {
                                const int wi = widx_uvw<In::U, In::V, In::WN_>(In::WOFF, c, v, w0 + ww);
                                if (part) part[wi] = dwacc[ww]; else atomicAdd(&p.dW[wi], dwacc[ww]);
                            }
                    }
                    }   // w0 tiles
#endif
                }
            }
        });
    }
}

// dW[i] (+)= sum over the chunks of the partial sums written by oeq_generic_backward_shared, in a fixed order: a block
// takes 32 weights; its 8 warps each add one eighth of the chunks in chunk order, and the eight sub-totals are added in
// warp order.  The order depends on the number of chunks only, so the result is bitwise reproducible.
extern "C" __global__ void __launch_bounds__(256) oeq_generic_dw_reduce(const T* __restrict__ part, long long chunks, T* __restrict__ dW, int accum) {
    __shared__ T sub[8][32];
    const int lane = threadIdx.x & 31, seg = threadIdx.x >> 5;
    const long long i = blockIdx.x * 32LL + lane;
    const long long per = (chunks + 7) / 8, c0 = seg * per, c1 = (c0 + per < chunks) ? c0 + per : chunks;
    T acc = T(0);
    if (i < WN) {
        long long c = c0;
        for (; c + 8 <= c1; c += 8) {
            T v[8];
#pragma unroll
            for (int q = 0; q < 8; ++q) v[q] = part[(c + q) * (long long)WN + i];
#pragma unroll
            for (int q = 0; q < 8; ++q) acc += v[q];
        }
        for (; c < c1; ++c) acc += part[c * (long long)WN + i];
    }
    sub[seg][lane] = acc;
    __syncthreads();
    if (seg == 0 && i < WN) {
        T tot = accum ? dW[i] : T(0);
#pragma unroll
        for (int q = 0; q < 8; ++q) tot += sub[q][lane];
        dW[i] = tot;
    }
}
#endif  // OEQ_SHARED_W

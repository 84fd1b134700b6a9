// Shared device helpers for the runtime-specialised kernels.
//
// Every translation unit handed to NVRTC is:   <problem header emitted from the descriptor>
//                                              + this file + one kernel file.
// The problem header defines:
//   typedef ... T;                       element type (float | double)
//   typedef ... IDX;                     index type of rows / cols / perm (long long | int)
//   OEQ_SHARED_W, OEQ_UVW, OEQ_IR_MUL, OEQ_KAHAN   0/1 switches
//   L1_DIM, L2_DIM, L3_DIM, WN, NINS, NB1, NB2, NB3   sizes
//   template<int> struct Blk1 / Blk2 / Blk3   { MUL, D, OFF }        feature blocks
//   template<int> struct Ins                  { A, B, O, WOFF, U, V, WN_, D1, D2, D3, fwd(), dx(), dy() }
//
// No system headers are included: NVRTC's built-in declarations suffice.
#pragma once

#ifndef OEQ_DEV
#define OEQ_DEV __device__ __forceinline__
#endif

// ---- compile-time loops -------------------------------------------------------------------------------------
template <int I> struct IntC { static constexpr int value = I; };
template <int I, int N, typename F>
OEQ_DEV void static_for(F&& f) {
    if constexpr (I < N) { f(IntC<I>{}); static_for<I + 1, N>(f); }
}

// ---- feature addressing -----------------------------------------------------------------------------------
// Element (u, i) of a block with multiplicity MUL and dimension D starting at OFF, in either layout.
template <int OFF, int MUL, int D>
OEQ_DEV int feat_idx(int u, int i) {
#if OEQ_IR_MUL
    return OFF + i * MUL + u;
#else
    return OFF + u * D + i;
#endif
}

// ---- weight addressing (kernel order: 32-wide tiles, [v][u] / [v][u][w] inside a tile) -------------------
template <int U, int V>
OEQ_DEV int widx_uvu(int woff, int u, int v) {
    if (U <= 32 && V <= 32) return woff + v * U + u;
    const int uc = u >> 5, ul = u & 31, vc = v >> 5, vl = v & 31;
    const int ulen = (U - (uc << 5)) < 32 ? (U - (uc << 5)) : 32;
    return woff + (uc << 5) * V + ulen * (vc << 5) + vl * ulen + ul;
}

template <int U, int V, int W>
OEQ_DEV int widx_uvw(int woff, int u, int v, int w) {
    if (U <= 32 && V <= 32 && W <= 32) return woff + (v * U + u) * W + w;
    const int uc = u >> 5, ul = u & 31, vc = v >> 5, vl = v & 31, wc = w >> 5, wl = w & 31;
    const int ulen = (U - (uc << 5)) < 32 ? (U - (uc << 5)) : 32;
    const int vlen = (V - (vc << 5)) < 32 ? (V - (vc << 5)) : 32;
    const int wlen = (W - (wc << 5)) < 32 ? (W - (wc << 5)) : 32;
    return woff + (uc << 5) * V * W + ulen * (vc << 5) * W + ulen * vlen * (wc << 5) + (vl * ulen + ul) * wlen + wl;
}

// ---- small utilities --------------------------------------------------------------------------------------
template <typename R>
OEQ_DEV R warp_sum(R v) {
#pragma unroll
    for (int s = 16; s > 0; s >>= 1) v += __shfl_xor_sync(0xffffffffu, v, s);
    return v;
}

// first index k in [0, n) with key(k) >= target, for a non-decreasing key
template <typename KeyFn>
OEQ_DEV long long lower_bound_ll(long long n, long long target, KeyFn key) {
    long long lo = 0, hi = n;
    while (lo < hi) {
        const long long mid = (lo + hi) >> 1;
        if ((long long)key(mid) < target) lo = mid + 1; else hi = mid;
    }
    return lo;
}

// output write modes
#define OEQ_OUT_STORE 0
#define OEQ_OUT_ADD 1
#define OEQ_OUT_ATOMIC 2

template <typename R>
OEQ_DEV void emit_out(R* p, R v, int mode) {
    if (mode == OEQ_OUT_STORE) *p = v;
    else if (mode == OEQ_OUT_ADD) *p += v;
    else atomicAdd(p, v);
}

// Per-row epilogue shared by every kernel: residual add, RMSNorm and FP8 quantisation with
// the rounding points of the PyTorch operator sequence in gpuk/__init__.py:147-173
// (allreduce_add_rms_native), which is the parity definition:
//
//   r  = T(sum + residual)                    -> residual_out          (:157)
//   n1 = T(float(r) * rsqrt(mean(r^2) + eps))                          (:152-154)
//   n  = T(float(w) * float(n1))              -> norm_out if no quant  (:155)
//   scale = max|n| / fp8_max  (fp32; 1 for an all-zero row)            (:160-161; impl.h:217)
//   q  = e4m3(clamp(float(n) / scale, +-fp8_max))                      (:162-164)
//
// The reference's fused kernel (src/impl/all_reduce_fusion_impl.h:159-228) keeps fp32 between
// those steps and therefore differs from its own PyTorch path by up to 1e-2 in the scales;
// this epilogue reproduces the PyTorch path instead.
//
// One CTA owns a row.  Thread t holds vectors t, t+B, t+2B, ... (B = blockDim.x) of the row
// so that every warp-wide access is one contiguous 512-byte segment.  The row stays packed in
// registers between the passes; the arithmetic is kept to ~14 instructions per element so
// that the kernels stay memory-bound: packed multiplies where the packed result rounds
// identically, and the division by the row's scale done as reciprocal + one exact-residual
// correction (q = n*y; q += fma(-q, scale, n) * y with y = 1/scale), which returns the
// correctly rounded quotient.
#pragma once

#include "common.cuh"

namespace gpuk {

struct EpilogueArgs {
    const void *residual;   // [rows, hidden] T
    const void *gamma;      // [hidden] T
    void *residual_out;     // [rows, hidden] T
    void *norm_out;         // [rows, hidden] T or FP8 bytes
    float *scale_out;       // dynamic: [rows] written; static: [1] read
    int hidden;             // elements per row
    int row_vecs;           // hidden / Elem<T>::kVec
    float eps;
    Quant q;
};

// Shared memory for the two block reductions of a row, double-buffered by row parity so
// that consecutive rows need no extra barrier between them.
struct alignas(16) EpilogueSmem {
    float red[2][2][32];
};

// The RMSNorm weight is re-read for every row (it stays in L1/L2) instead of being held in
// registers across rows: that keeps the register footprint low enough for four 256-thread
// CTAs per SM.  Loads are issued before the first block reduction so their latency is hidden.
template <typename T, int VPT>
__device__ __forceinline__ void load_gamma(const EpilogueArgs &a, uint4 (&g)[VPT]) {
#pragma unroll
    for (int i = 0; i < VPT; ++i) {
        const int v = threadIdx.x + i * blockDim.x;
        g[i] = v < a.row_vecs ? ld_keep(reinterpret_cast<const uint4 *>(a.gamma) + v) : make_uint4(0, 0, 0, 0);
    }
}

// Issues the loads of this thread's residual vectors of `row` (all in flight together).
template <typename T, int VPT>
__device__ __forceinline__ void load_residual(const EpilogueArgs &a, int64_t row, uint4 (&res)[VPT]) {
    const uint4 *src = reinterpret_cast<const uint4 *>(a.residual) + row * a.row_vecs;
#pragma unroll
    for (int i = 0; i < VPT; ++i) {
        const int v = threadIdx.x + i * blockDim.x;
        res[i] = v < a.row_vecs ? ld_stream(src + v) : make_uint4(0, 0, 0, 0);
    }
}

// `x[i]` holds the all-reduced sum (already rounded to T) and `res[i]` the residual for vector
// threadIdx.x + i*blockDim.x of row `row` (zeros beyond the row); on return the row's
// residual_out / norm_out / scale_out have been written.
template <typename T, int VPT>
__device__ __forceinline__ void row_epilogue(const EpilogueArgs &a, int64_t row, uint4 (&x)[VPT],
                                             const uint4 (&res)[VPT], EpilogueSmem &sm, int parity,
                                             float static_scale) {
    constexpr int KV = Elem<T>::kVec;
    const int64_t row_base = row * a.row_vecs;
    float ss = 0.f;
    // r = T(sum + residual); kept packed in x
#pragma unroll
    for (int i = 0; i < VPT; ++i) {
        const int v = threadIdx.x + i * blockDim.x;
        float r[KV];
        x[i] = Elem<T>::add(x[i], res[i]);
        if (v < a.row_vecs) st_stream(reinterpret_cast<uint4 *>(a.residual_out) + row_base + v, x[i]);
        Elem<T>::unpack(x[i], r);
#pragma unroll
        for (int e = 0; e < KV; ++e) ss = fmaf(r[e], r[e], ss);
    }
    uint4 g[VPT];
    load_gamma<T, VPT>(a, g);
    ss = block_sum(ss, sm.red[parity][0]);
    const float rstd = 1.0f / sqrtf(ss / static_cast<float>(a.hidden) + a.eps);

    typename Elem<T>::AbsMax am = Elem<T>::absmax_init();
#pragma unroll
    for (int i = 0; i < VPT; ++i) {
        const int v = threadIdx.x + i * blockDim.x;
        float r[KV];
        Elem<T>::unpack(x[i], r);
#pragma unroll
        for (int e = 0; e < KV; ++e) r[e] *= rstd;
        x[i] = Elem<T>::mul(g[i], Elem<T>::pack(r));
        Elem<T>::absmax_update(am, x[i]);
        if (a.q.mode == kQuantNone && v < a.row_vecs)
            st_stream(reinterpret_cast<uint4 *>(a.norm_out) + row_base + v, x[i]);
    }
    if (a.q.mode == kQuantNone) return;

    float scale = static_scale;
    if (a.q.mode == kQuantDynamic) {
        const float amax = block_max(Elem<T>::absmax_value(am), sm.red[parity][1]);
        scale = amax == 0.f ? 1.f : amax / a.q.fp8_max;
        if (threadIdx.x == 0) a.scale_out[row] = scale;
    }
    // |n / scale| <= fp8_max by construction for the dynamic policies and the static policy
    // saturates at the format maximum, so the saturating convert is the clamp.
    const float y = 1.0f / scale;
#pragma unroll
    for (int i = 0; i < VPT; ++i) {
        const int v = threadIdx.x + i * blockDim.x;
        float n[KV], q[KV];
        Elem<T>::unpack(x[i], n);
#pragma unroll
        for (int e = 0; e < KV; ++e) {
            q[e] = n[e] * y;
            q[e] = copysignf(fmaf(fmaf(-q[e], scale, n[e]), y, q[e]), n[e]);   // keeps the sign of a zero
        }
        if (v < a.row_vecs) {
            uint8_t *dst = reinterpret_cast<uint8_t *>(a.norm_out) + (row_base + v) * KV;
            if constexpr (KV == 8) {
                uint2 o;
                o.x = cvt_e4m3x4(q[0], q[1], q[2], q[3], a.q.fnuz);
                o.y = cvt_e4m3x4(q[4], q[5], q[6], q[7], a.q.fnuz);
                __stcs(reinterpret_cast<uint2 *>(dst), o);
            } else {
                __stcs(reinterpret_cast<uint32_t *>(dst), cvt_e4m3x4(q[0], q[1], q[2], q[3], a.q.fnuz));
            }
        }
    }
}

}  // namespace gpuk

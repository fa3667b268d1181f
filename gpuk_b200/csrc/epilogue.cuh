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
// One CTA owns a row, or -- where few rows must be spread over many SMs -- one contiguous
// segment of a row, the other segments being held by the other CTAs of its thread-block
// cluster (the two row-wide reductions then take one extra hop through distributed shared
// memory).  Thread t holds vectors v0+t, v0+t+B, v0+t+2B, ... (B = blockDim.x) of its segment
// [v0, v1) so that every warp-wide access is one contiguous 512-byte piece.  The row stays packed in
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

// The part of a row one CTA works on, and the CTA's place in the cluster that holds the row.
struct RowSeg {
    int v0, v1;     // vectors [v0, v1) of the row
    int cl_rank;    // this CTA's rank in the cluster
    int cl_size;    // CTAs per row (1: the CTA holds the whole row)
};
__device__ __forceinline__ RowSeg whole_row(int row_vecs) { return RowSeg{0, row_vecs, 0, 1}; }

// Shared memory for the two block reductions of a row (and their cluster stage), double-
// buffered by row parity so that consecutive rows need no extra barrier between them.
struct alignas(16) EpilogueSmem {
    float red[2][2][32];
    float cl[2][2][8];
    unsigned long long seq;   // number of the running exchange, fetched once per CTA (begin_call)
};

// The RMSNorm weight is re-read for every row (it stays in L1/L2) instead of being held in
// registers across rows: that keeps the register footprint low enough for four 256-thread
// CTAs per SM.  Loads are issued before the first block reduction so their latency is hidden.
template <typename T, int VPT>
__device__ __forceinline__ void load_gamma(const EpilogueArgs &a, const RowSeg &seg, uint4 (&g)[VPT]) {
#pragma unroll
    for (int i = 0; i < VPT; ++i) {
        const int v = seg.v0 + threadIdx.x + i * blockDim.x;
        g[i] = v < seg.v1 ? ld_keep(reinterpret_cast<const uint4 *>(a.gamma) + v) : make_uint4(0, 0, 0, 0);
    }
}

// Issues the loads of this thread's residual vectors of `row` (all in flight together).
template <typename T, int VPT>
__device__ __forceinline__ void load_residual(const EpilogueArgs &a, const RowSeg &seg, int64_t row, uint4 (&res)[VPT]) {
    const uint4 *src = reinterpret_cast<const uint4 *>(a.residual) + row * a.row_vecs;
#pragma unroll
    for (int i = 0; i < VPT; ++i) {
        const int v = seg.v0 + threadIdx.x + i * blockDim.x;
        res[i] = v < seg.v1 ? ld_stream(src + v) : make_uint4(0, 0, 0, 0);
    }
}

// `x[i]` holds the all-reduced sum (already rounded to T) and `res[i]` the residual for vector
// seg.v0 + threadIdx.x + i*blockDim.x of row `row` (zeros beyond the segment); on return this
// segment of the row's residual_out / norm_out and the row's scale_out have been written.
// Every thread of every CTA of the cluster must call it for the same row.  `after_sum` runs in
// every thread right after the first block-wide reduction, i.e. once all threads of the CTA
// have consumed their inputs (the staged kernel refills its shared-memory stage there).
struct NoHook {
    __device__ __forceinline__ void operator()() const {}
};
template <typename T, int VPT, typename Hook = NoHook>
__device__ __forceinline__ void row_epilogue(const EpilogueArgs &a, const RowSeg &seg, int64_t row, uint4 (&x)[VPT],
                                             const uint4 (&res)[VPT], EpilogueSmem &sm, int parity,
                                             float static_scale, Hook after_sum = Hook()) {
    constexpr int KV = Elem<T>::kVec;
    const int64_t row_base = row * a.row_vecs;
    float ss = 0.f;
    // r = T(sum + residual); kept packed in x
#pragma unroll
    for (int i = 0; i < VPT; ++i) {
        const int v = seg.v0 + threadIdx.x + i * blockDim.x;
        float r[KV];
        x[i] = Elem<T>::add(x[i], res[i]);
        if (v < seg.v1) st_stream(reinterpret_cast<uint4 *>(a.residual_out) + row_base + v, x[i]);
        Elem<T>::unpack(x[i], r);
#pragma unroll
        for (int e = 0; e < KV; ++e) ss = fmaf(r[e], r[e], ss);
    }
    uint4 g[VPT];
    load_gamma<T, VPT>(a, seg, g);
    ss = block_sum(ss, sm.red[parity][0]);
    after_sum();
    ss = cluster_combine<false>(ss, sm.cl[parity][0], seg.cl_rank, seg.cl_size);
    const float rstd = 1.0f / sqrtf(ss / static_cast<float>(a.hidden) + a.eps);

    typename Elem<T>::AbsMax am = Elem<T>::absmax_init();
#pragma unroll
    for (int i = 0; i < VPT; ++i) {
        const int v = seg.v0 + threadIdx.x + i * blockDim.x;
        float r[KV];
        Elem<T>::unpack(x[i], r);
#pragma unroll
        for (int e = 0; e < KV; ++e) r[e] *= rstd;
        x[i] = Elem<T>::mul(g[i], Elem<T>::pack(r));
        Elem<T>::absmax_update(am, x[i]);
        if (a.q.mode == kQuantNone && v < seg.v1)
            st_stream(reinterpret_cast<uint4 *>(a.norm_out) + row_base + v, x[i]);
    }
    if (a.q.mode == kQuantNone) return;

    float scale = static_scale;
    if (a.q.mode == kQuantDynamic) {
        float amax = block_max(Elem<T>::absmax_value(am), sm.red[parity][1]);
        amax = cluster_combine<true>(amax, sm.cl[parity][1], seg.cl_rank, seg.cl_size);
        scale = amax == 0.f ? 1.f : amax / a.q.fp8_max;
        if (threadIdx.x == 0 && seg.cl_rank == 0) a.scale_out[row] = scale;
    }
    // |n / scale| <= fp8_max by construction for the dynamic policies and the static policy
    // saturates at the format maximum, so the saturating convert is the clamp.
    const float y = 1.0f / scale;
#pragma unroll
    for (int i = 0; i < VPT; ++i) {
        const int v = seg.v0 + threadIdx.x + i * blockDim.x;
        float n[KV], q[KV];
        Elem<T>::unpack(x[i], n);
#pragma unroll
        for (int e = 0; e < KV; ++e) {
            q[e] = n[e] * y;
            q[e] = copysignf(fmaf(fmaf(-q[e], scale, n[e]), y, q[e]), n[e]);   // keeps the sign of a zero
        }
        if (v < seg.v1) {
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

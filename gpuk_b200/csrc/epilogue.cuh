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

#include <type_traits>

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
    float hidden_f;         // float(hidden) and its correctly rounded reciprocal
    float inv_hidden;
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
    int rows_finished;        // warp-specialised two-shot kernel: rows this CTA's finishing warps have completed
};

// The RMSNorm weight is re-read for every row (it stays in L1/L2) instead of being held in
// registers across rows: that keeps the register footprint low enough for four 256-thread
// CTAs per SM.  Loads are issued before the first block reduction so their latency is hidden.
template <typename T, int VPT, bool FULL = false>
__device__ __forceinline__ void load_gamma(const EpilogueArgs &a, const RowSeg &seg, const Group &grp, uint4 (&g)[VPT]) {
#pragma unroll
    for (int i = 0; i < VPT; ++i) {
        const int v = seg.v0 + grp.tid + i * grp.n;
        g[i] = (FULL || v < seg.v1) ? ld_keep(reinterpret_cast<const uint4 *>(a.gamma) + v) : make_uint4(0, 0, 0, 0);
    }
}

// Issues the loads of this thread's residual vectors of `row` (all in flight together).
template <typename T, int VPT, bool FULL = false>
__device__ __forceinline__ void load_residual(const EpilogueArgs &a, const RowSeg &seg, int64_t row, const Group &grp, uint4 (&res)[VPT]) {
    const uint4 *src = reinterpret_cast<const uint4 *>(a.residual) + row * a.row_vecs;
#pragma unroll
    for (int i = 0; i < VPT; ++i) {
        const int v = seg.v0 + grp.tid + i * grp.n;
        res[i] = (FULL || v < seg.v1) ? ld_stream(src + v) : make_uint4(0, 0, 0, 0);
    }
}

// Correctly rounded a / b for a divisor known ahead of time (inv_b = RN(1 / b)): a multiplication
// and two fused corrections instead of the generic division sequence.  q0 = RN(a * inv_b) is within
// one unit of the quotient, r = a - q0 * b is exact in one FMA, and RN(q0 + r * inv_b) is the
// correctly rounded quotient (Markstein).  Falls back to the division where the exact residual
// could underflow.
__device__ __forceinline__ float div_by_known(float a, float b, float inv_b) {
    if (fabsf(a) < 1e-30f) return a / b;
    const float q0 = a * inv_b;
    return fmaf(fmaf(-q0, b, a), inv_b, q0);
}

// `x[i]` holds the all-reduced sum (already rounded to T) and `res[i]` the residual for vector
// seg.v0 + grp.tid + i*grp.n of row `row` (zeros beyond the segment); on return this
// segment of the row's residual_out / norm_out and the row's scale_out have been written.
// Every thread of the group `grp` (the whole CTA, or the finishing warps of a warp-specialised
// kernel) in every CTA of the cluster must call it for the same row.  `after_sum` runs in every
// thread right after the first group-wide reduction, i.e. once all threads of the group have
// consumed their inputs (the staged kernel refills its shared-memory stage there).
// FULL: every thread's VPT vectors lie inside the segment (no bounds checks are compiled in).
//
// Arithmetic per pair of elements, all of it on packed registers: one packed add (residual), two
// integer operations to widen to an fp32 pair, one packed fp32 FMA (sum of squares), one packed
// fp32 multiply (by rstd), one rounding convert, one packed multiply (weight), two operations for
// the running |max|, two to widen again, three packed fp32 operations for the correctly rounded
// division by the scale, and half an FP8 convert.
struct NoHook {
    __device__ __forceinline__ void operator()() const {}
};
template <typename T, int VPT, bool FULL = false, typename Hook = NoHook>
__device__ __forceinline__ void row_epilogue(const EpilogueArgs &a, const RowSeg &seg, int64_t row, const Group &grp,
                                             uint4 (&x)[VPT], const uint4 (&res)[VPT], EpilogueSmem &sm, int parity,
                                             float static_scale, Hook after_sum = Hook()) {
    constexpr int KV = Elem<T>::kVec;
    constexpr int NP = Elem<T>::kPairs;
    const int64_t row_base = row * a.row_vecs;
    const int vbase = seg.v0 + grp.tid;
    auto inside = [&](int i) { return FULL || vbase + i * grp.n < seg.v1; };
    // r = T(sum + residual), kept packed in x; sum of squares in two packed accumulators
    f32x2 ssa = 0ull, ssb = 0ull;
    uint4 *ro = reinterpret_cast<uint4 *>(a.residual_out) + row_base + vbase;
#pragma unroll
    for (int i = 0; i < VPT; ++i) {
        x[i] = Elem<T>::add(x[i], res[i]);
        if (inside(i)) st_stream(ro + i * grp.n, x[i]);
        f32x2 p[NP];
        Elem<T>::unpack2(x[i], p);
#pragma unroll
        for (int k = 0; k < NP; k += 2) {
            ssa = f2_fma(p[k], p[k], ssa);
            ssb = f2_fma(p[k + 1], p[k + 1], ssb);
        }
    }
    uint4 g[VPT];
    load_gamma<T, VPT, FULL>(a, seg, grp, g);
    float ss = block_sum(f2_sum(f2_add(ssa, ssb)), sm.red[parity][0], grp);
    after_sum();
    ss = cluster_combine<false>(ss, sm.cl[parity][0], seg.cl_rank, seg.cl_size);
    const float rstd = 1.0f / sqrtf(div_by_known(ss, a.hidden_f, a.inv_hidden) + a.eps);
    const f32x2 rstd2 = f2_splat(rstd);

    typename Elem<T>::AbsMax am = Elem<T>::absmax_init();
    uint4 *no = reinterpret_cast<uint4 *>(a.norm_out) + row_base + vbase;
#pragma unroll
    for (int i = 0; i < VPT; ++i) {
        f32x2 p[NP];
        Elem<T>::unpack2(x[i], p);
#pragma unroll
        for (int k = 0; k < NP; ++k) p[k] = f2_mul(p[k], rstd2);
        x[i] = Elem<T>::mul(g[i], Elem<T>::pack2(p));
        Elem<T>::absmax_update(am, x[i]);
        if (a.q.mode == kQuantNone && inside(i)) st_stream(no + i * grp.n, x[i]);
    }
    if (a.q.mode == kQuantNone) return;

    float scale = static_scale;
    if (a.q.mode == kQuantDynamic) {
        float amax = block_max(Elem<T>::absmax_value(am), sm.red[parity][1], grp);
        amax = cluster_combine<true>(amax, sm.cl[parity][1], seg.cl_rank, seg.cl_size);
        scale = amax == 0.f ? 1.f : div_by_known(amax, a.q.fp8_max, a.q.inv_fp8_max);
        if (grp.tid == 0 && seg.cl_rank == 0) a.scale_out[row] = scale;
    }
    // q = n / scale, correctly rounded, as y = 1 / scale, q0 = n * y, q = q0 + (n - q0 * scale) * y.
    // |q| <= fp8_max by construction for the dynamic policies and the static policy saturates at the
    // format maximum, so the saturating convert is the clamp.  For the fnuz flavour the quotient is
    // doubled on the way (its exponent bias is 8 where e4m3fn has 7, so code_fnuz(v) = code_fn(2v)):
    // y is doubled and the scale halved, both exact.  The sign of every byte is taken from n itself
    // (a negative zero keeps its sign, as in the division), and fnuz then folds 0x80, its NaN, to 0.
    const float y = (a.q.fnuz ? 2.0f : 1.0f) / scale;
    const f32x2 y2 = f2_splat(y);
    const f32x2 neg_s2 = f2_splat(a.q.fnuz ? -0.5f * scale : -scale);
    uint8_t *qo = reinterpret_cast<uint8_t *>(a.norm_out) + (row_base + vbase) * KV;
    auto quantise = [&](auto fnuz_tag) {
        constexpr bool FNUZ = decltype(fnuz_tag)::value;
#pragma unroll
        for (int i = 0; i < VPT; ++i) {
            f32x2 p[NP];
            Elem<T>::unpack2(x[i], p);
            uint32_t out[NP / 2];
#pragma unroll
            for (int k = 0; k < NP; k += 2) {
                f32x2 q0 = f2_mul(p[k], y2), q1 = f2_mul(p[k + 1], y2);
                q0 = f2_fma(f2_fma(q0, neg_s2, p[k]), y2, q0);
                q1 = f2_fma(f2_fma(q1, neg_s2, p[k + 1]), y2, q1);
                const uint32_t w = (cvt_e4m3x4_pairs(q0, q1) & 0x7f7f7f7fu) | Elem<T>::sign_bytes(x[i], k / 2);
                out[k / 2] = FNUZ ? fold_negative_zero_bytes(w) : w;
            }
            if (inside(i)) {
                uint8_t *dst = qo + static_cast<size_t>(i) * grp.n * KV;
                if constexpr (KV == 8) __stcs(reinterpret_cast<uint2 *>(dst), make_uint2(out[0], out[1]));
                else __stcs(reinterpret_cast<uint32_t *>(dst), out[0]);
            }
        }
    };
    if (a.q.fnuz) quantise(std::true_type());
    else quantise(std::false_type());
}

}  // namespace gpuk

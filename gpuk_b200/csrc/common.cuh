// Device-side building blocks shared by every kernel of the tensor-parallel epilogue:
// 16-byte vector access, element traits with explicit rounding, warp/block reductions,
// the hardware FP8 cast, and the cross-GPU hand-off primitives with bounded waits.
//
// Replaces, for sm_100a only, the reference's src/common/kernel_utils.h:29-99 (vec_t,
// warp_reduce, block_reduce), src/common/communicator.h:12-36,79-113 (st_flag, ld_flag,
// SyncComm) and the software FP8 cast of src/common/float8.h:17-150.
#pragma once

#include <cuda_bf16.h>
#include <cuda_fp16.h>
#include <cuda_runtime.h>
#include <stdint.h>

namespace gpuk {

constexpr int kMaxRanks = 8;        // communicator.h:57
constexpr int kMaxBlocks = 2048;    // upper bound on CTAs per rank (reference: 80, communicator.h:58)
constexpr int kStatusWords = 8;

// ---------------------------------------------------------------------------------------
// quantisation policy (host picks it from the operator's quant_type argument)
// ---------------------------------------------------------------------------------------
enum QuantMode : int { kQuantNone = 0, kQuantDynamic = 1, kQuantStatic = 2 };

struct Quant {
    int mode;        // QuantMode
    int fnuz;        // 1: e4m3fnuz bit patterns (bias 8, no negative zero), 0: e4m3fn
    float fp8_max;   // saturation value used for the scale and the clamp (240 / 120 / 448)
    float inv_fp8_max;   // its correctly rounded reciprocal
};
__host__ __device__ inline Quant make_quant(int mode, int fnuz, float fp8_max) {
    Quant q;
    q.mode = mode;
    q.fnuz = fnuz;
    q.fp8_max = fp8_max;
    q.inv_fp8_max = fp8_max > 0.f ? static_cast<float>(1.0 / static_cast<double>(fp8_max)) : 0.f;
    return q;
}

// ---------------------------------------------------------------------------------------
// device-resident state of one rank's workspace (local, never mapped by peers)
// ---------------------------------------------------------------------------------------
struct LocalState {
    unsigned long long seq;   // bits 63..16: exchanges completed so far (the low bit of that number selects the
                              // staging buffer of the next one); bits 15..0: tickets taken by CTAs of the running call
    uint32_t reserved2;
    uint32_t abort;       // set once a wait has run out, so that later waits give up at once
    unsigned long long timeout_ns;
    uint32_t status[kStatusWords];   // [0]=code (0 ok), [1]=rank, [2]=CTA, [3]=stage, [4]=peer, [5]=thread, [6]=word seen
};

// stage codes in status[3]
enum Stage : int { kStageOneShot = 0, kStageScatter = 1, kStageGather = 2, kStageSelfTest = 3, kStageSymIn = 4, kStageSymOut = 5,
                   kStageReady = 6 };   // waiting for the producer of this rank's own input (row-block ready words)

// kStatusClusterMismatch: the kernel found itself in a thread-block cluster of another size than the
// host planned (status[6] = the size seen); it returns before it takes a ticket or writes anything.
enum StatusCode : uint32_t { kStatusOk = 0, kStatusWaitTimeout = 1, kStatusSpinCap = 2, kStatusClusterMismatch = 3 };

// ---------------------------------------------------------------------------------------
// 16-byte global memory access
// ---------------------------------------------------------------------------------------
// Streaming read of data that is read once (inputs, residual): evict-first.
__device__ __forceinline__ uint4 ld_stream(const void *p) { return __ldcs(reinterpret_cast<const uint4 *>(p)); }
// Read of staging memory that a peer GPU has written: served by L2, never by a stale L1 line.
__device__ __forceinline__ uint4 ld_staging(const void *p) { return __ldcg(reinterpret_cast<const uint4 *>(p)); }
// Read-mostly data with reuse across rows (RMSNorm weight).
__device__ __forceinline__ uint4 ld_keep(const void *p) { return __ldg(reinterpret_cast<const uint4 *>(p)); }
__device__ __forceinline__ void st_stream(void *p, const uint4 &v) { __stcs(reinterpret_cast<uint4 *>(p), v); }
// Store into memory that may live on a peer GPU (or locally): plain write-back store.
__device__ __forceinline__ void st_peer(void *p, const uint4 &v) { *reinterpret_cast<uint4 *>(p) = v; }

// ---------------------------------------------------------------------------------------
// packed fp32 pairs: sm_100 multiplies and fuses two fp32 lanes held in one 64-bit register
// pair with ONE instruction (mul / add / fma .f32x2, each lane rounded like the scalar form),
// which halves the issue slots of the per-element arithmetic.  .x is the low lane.
// ---------------------------------------------------------------------------------------
using f32x2 = unsigned long long;
__device__ __forceinline__ f32x2 f2_make(float lo, float hi) {
    f32x2 r;
    asm("mov.b64 %0, {%1, %2};" : "=l"(r) : "f"(lo), "f"(hi));
    return r;
}
__device__ __forceinline__ f32x2 f2_make_bits(uint32_t lo, uint32_t hi) {
    f32x2 r;
    asm("mov.b64 %0, {%1, %2};" : "=l"(r) : "r"(lo), "r"(hi));
    return r;
}
__device__ __forceinline__ f32x2 f2_splat(float v) { return f2_make(v, v); }
__device__ __forceinline__ void f2_split(f32x2 v, float &lo, float &hi) {
    asm("mov.b64 {%0, %1}, %2;" : "=f"(lo), "=f"(hi) : "l"(v));
}
__device__ __forceinline__ f32x2 f2_mul(f32x2 a, f32x2 b) {
    f32x2 r;
    asm("mul.rn.f32x2 %0, %1, %2;" : "=l"(r) : "l"(a), "l"(b));
    return r;
}
__device__ __forceinline__ f32x2 f2_add(f32x2 a, f32x2 b) {
    f32x2 r;
    asm("add.rn.f32x2 %0, %1, %2;" : "=l"(r) : "l"(a), "l"(b));
    return r;
}
__device__ __forceinline__ f32x2 f2_fma(f32x2 a, f32x2 b, f32x2 c) {
    f32x2 r;
    asm("fma.rn.f32x2 %0, %1, %2, %3;" : "=l"(r) : "l"(a), "l"(b), "l"(c));
    return r;
}
__device__ __forceinline__ float f2_sum(f32x2 v) {
    float lo, hi;
    f2_split(v, lo, hi);
    return lo + hi;
}

// ---------------------------------------------------------------------------------------
// element traits: how 16 bytes unpack to fp32 lanes and round back
// ---------------------------------------------------------------------------------------
template <typename T>
struct Elem;

template <>
struct Elem<__nv_bfloat16> {
    static constexpr int kVec = 8;
    static constexpr int kPairs = 4;
    // the 16 bytes as four fp32 pairs (elements 2k, 2k+1), and back with one rounding per element
    __device__ static __forceinline__ void unpack2(const uint4 &u, f32x2 (&p)[4]) {
        const uint32_t w[4] = {u.x, u.y, u.z, u.w};
#pragma unroll
        for (int i = 0; i < 4; ++i) p[i] = f2_make_bits(w[i] << 16, w[i] & 0xffff0000u);
    }
    __device__ static __forceinline__ uint4 pack2(const f32x2 (&p)[4]) {
        uint32_t w[4];
#pragma unroll
        for (int i = 0; i < 4; ++i) {
            float lo, hi;
            f2_split(p[i], lo, hi);
            asm("cvt.rn.bf16x2.f32 %0, %1, %2;" : "=r"(w[i]) : "f"(hi), "f"(lo));
        }
        return make_uint4(w[0], w[1], w[2], w[3]);
    }
    // sign bits of elements 4h .. 4h+3 at bits 7, 15, 23, 31
    __device__ static __forceinline__ uint32_t sign_bytes(const uint4 &u, int h) {
        return __byte_perm(h ? u.z : u.x, h ? u.w : u.y, 0x7531) & 0x80808080u;
    }
    __device__ static __forceinline__ void unpack(const uint4 &u, float (&f)[8]) {
        const uint32_t w[4] = {u.x, u.y, u.z, u.w};
#pragma unroll
        for (int i = 0; i < 4; ++i) {
            f[2 * i] = __uint_as_float(w[i] << 16);
            f[2 * i + 1] = __uint_as_float(w[i] & 0xffff0000u);
        }
    }
    __device__ static __forceinline__ uint4 pack(const float (&f)[8]) {
        uint32_t w[4];
#pragma unroll
        for (int i = 0; i < 4; ++i) {
            __nv_bfloat162 h = __floats2bfloat162_rn(f[2 * i], f[2 * i + 1]);
            w[i] = *reinterpret_cast<uint32_t *>(&h);
        }
        return make_uint4(w[0], w[1], w[2], w[3]);
    }
    // elementwise T(a * b): the product of two bf16 values is exact in fp32, so one packed
    // multiply rounds exactly like "convert, multiply in fp32, round"
    __device__ static __forceinline__ uint4 mul(const uint4 &a, const uint4 &b) {
        const uint32_t wa[4] = {a.x, a.y, a.z, a.w}, wb[4] = {b.x, b.y, b.z, b.w};
        uint32_t w[4];
#pragma unroll
        for (int i = 0; i < 4; ++i) {
            __nv_bfloat162 h = __hmul2(*reinterpret_cast<const __nv_bfloat162 *>(&wa[i]),
                                       *reinterpret_cast<const __nv_bfloat162 *>(&wb[i]));
            w[i] = *reinterpret_cast<uint32_t *>(&h);
        }
        return make_uint4(w[0], w[1], w[2], w[3]);
    }
    // elementwise T(a + b).  The fp32 sum of two bf16 values is either exact (exponents at most
    // 16 apart) or dominated by the larger operand, so a packed add with one rounding gives
    // the same bits as "convert, add in fp32, round".
    __device__ static __forceinline__ uint4 add(const uint4 &a, const uint4 &b) {
        const uint32_t wa[4] = {a.x, a.y, a.z, a.w}, wb[4] = {b.x, b.y, b.z, b.w};
        uint32_t w[4];
#pragma unroll
        for (int i = 0; i < 4; ++i) {
            __nv_bfloat162 h = __hadd2(*reinterpret_cast<const __nv_bfloat162 *>(&wa[i]),
                                       *reinterpret_cast<const __nv_bfloat162 *>(&wb[i]));
            w[i] = *reinterpret_cast<uint32_t *>(&h);
        }
        return make_uint4(w[0], w[1], w[2], w[3]);
    }
    // running maximum of magnitudes, kept as a packed pair
    using AbsMax = uint32_t;
    __device__ static __forceinline__ AbsMax absmax_init() { return 0u; }
    __device__ static __forceinline__ void absmax_update(AbsMax &m, const uint4 &a) {
        const uint32_t w[4] = {a.x, a.y, a.z, a.w};
#pragma unroll
        for (int i = 0; i < 4; ++i) {
            const uint32_t mag = w[i] & 0x7fff7fffu;
            __nv_bfloat162 h = __hmax2(*reinterpret_cast<const __nv_bfloat162 *>(&m),
                                       *reinterpret_cast<const __nv_bfloat162 *>(&mag));
            m = *reinterpret_cast<uint32_t *>(&h);
        }
    }
    __device__ static __forceinline__ float absmax_value(AbsMax m) {
        return fmaxf(__uint_as_float(m << 16), __uint_as_float(m & 0xffff0000u));
    }
};

template <>
struct Elem<__half> {
    static constexpr int kVec = 8;
    static constexpr int kPairs = 4;
    __device__ static __forceinline__ void unpack2(const uint4 &u, f32x2 (&p)[4]) {
        const uint32_t w[4] = {u.x, u.y, u.z, u.w};
#pragma unroll
        for (int i = 0; i < 4; ++i) {
            const float2 v = __half22float2(*reinterpret_cast<const __half2 *>(&w[i]));
            p[i] = f2_make(v.x, v.y);
        }
    }
    __device__ static __forceinline__ uint4 pack2(const f32x2 (&p)[4]) {
        uint32_t w[4];
#pragma unroll
        for (int i = 0; i < 4; ++i) {
            float lo, hi;
            f2_split(p[i], lo, hi);
            __half2 h = __floats2half2_rn(lo, hi);
            w[i] = *reinterpret_cast<uint32_t *>(&h);
        }
        return make_uint4(w[0], w[1], w[2], w[3]);
    }
    __device__ static __forceinline__ uint32_t sign_bytes(const uint4 &u, int h) {
        return __byte_perm(h ? u.z : u.x, h ? u.w : u.y, 0x7531) & 0x80808080u;
    }
    __device__ static __forceinline__ void unpack(const uint4 &u, float (&f)[8]) {
        const uint32_t w[4] = {u.x, u.y, u.z, u.w};
#pragma unroll
        for (int i = 0; i < 4; ++i) {
            float2 v = __half22float2(*reinterpret_cast<const __half2 *>(&w[i]));
            f[2 * i] = v.x;
            f[2 * i + 1] = v.y;
        }
    }
    __device__ static __forceinline__ uint4 pack(const float (&f)[8]) {
        uint32_t w[4];
#pragma unroll
        for (int i = 0; i < 4; ++i) {
            __half2 h = __floats2half2_rn(f[2 * i], f[2 * i + 1]);
            w[i] = *reinterpret_cast<uint32_t *>(&h);
        }
        return make_uint4(w[0], w[1], w[2], w[3]);
    }
    __device__ static __forceinline__ uint4 mul(const uint4 &a, const uint4 &b) {
        const uint32_t wa[4] = {a.x, a.y, a.z, a.w}, wb[4] = {b.x, b.y, b.z, b.w};
        uint32_t w[4];
#pragma unroll
        for (int i = 0; i < 4; ++i) {
            __half2 h = __hmul2(*reinterpret_cast<const __half2 *>(&wa[i]), *reinterpret_cast<const __half2 *>(&wb[i]));
            w[i] = *reinterpret_cast<uint32_t *>(&h);
        }
        return make_uint4(w[0], w[1], w[2], w[3]);
    }
    // same argument as for bf16: exact in fp32 up to 13 binades apart, dominated beyond
    __device__ static __forceinline__ uint4 add(const uint4 &a, const uint4 &b) {
        const uint32_t wa[4] = {a.x, a.y, a.z, a.w}, wb[4] = {b.x, b.y, b.z, b.w};
        uint32_t w[4];
#pragma unroll
        for (int i = 0; i < 4; ++i) {
            __half2 h = __hadd2(*reinterpret_cast<const __half2 *>(&wa[i]), *reinterpret_cast<const __half2 *>(&wb[i]));
            w[i] = *reinterpret_cast<uint32_t *>(&h);
        }
        return make_uint4(w[0], w[1], w[2], w[3]);
    }
    using AbsMax = uint32_t;
    __device__ static __forceinline__ AbsMax absmax_init() { return 0u; }
    __device__ static __forceinline__ void absmax_update(AbsMax &m, const uint4 &a) {
        const uint32_t w[4] = {a.x, a.y, a.z, a.w};
#pragma unroll
        for (int i = 0; i < 4; ++i) {
            const uint32_t mag = w[i] & 0x7fff7fffu;
            __half2 h = __hmax2(*reinterpret_cast<const __half2 *>(&m), *reinterpret_cast<const __half2 *>(&mag));
            m = *reinterpret_cast<uint32_t *>(&h);
        }
    }
    __device__ static __forceinline__ float absmax_value(AbsMax m) {
        const float2 v = __half22float2(*reinterpret_cast<const __half2 *>(&m));
        return fmaxf(v.x, v.y);
    }
};

template <>
struct Elem<float> {
    static constexpr int kVec = 4;
    static constexpr int kPairs = 2;
    __device__ static __forceinline__ void unpack2(const uint4 &u, f32x2 (&p)[2]) {
        p[0] = f2_make_bits(u.x, u.y);
        p[1] = f2_make_bits(u.z, u.w);
    }
    __device__ static __forceinline__ uint4 pack2(const f32x2 (&p)[2]) {
        float a, b, c, d;
        f2_split(p[0], a, b);
        f2_split(p[1], c, d);
        return make_uint4(__float_as_uint(a), __float_as_uint(b), __float_as_uint(c), __float_as_uint(d));
    }
    __device__ static __forceinline__ uint32_t sign_bytes(const uint4 &u, int) {
        return __byte_perm(__byte_perm(u.x, u.y, 0x7773), __byte_perm(u.z, u.w, 0x7773), 0x5410) & 0x80808080u;
    }
    __device__ static __forceinline__ void unpack(const uint4 &u, float (&f)[4]) {
        f[0] = __uint_as_float(u.x);
        f[1] = __uint_as_float(u.y);
        f[2] = __uint_as_float(u.z);
        f[3] = __uint_as_float(u.w);
    }
    __device__ static __forceinline__ uint4 pack(const float (&f)[4]) {
        return make_uint4(__float_as_uint(f[0]), __float_as_uint(f[1]), __float_as_uint(f[2]), __float_as_uint(f[3]));
    }
    __device__ static __forceinline__ uint4 mul(const uint4 &a, const uint4 &b) {
        return make_uint4(__float_as_uint(__uint_as_float(a.x) * __uint_as_float(b.x)),
                          __float_as_uint(__uint_as_float(a.y) * __uint_as_float(b.y)),
                          __float_as_uint(__uint_as_float(a.z) * __uint_as_float(b.z)),
                          __float_as_uint(__uint_as_float(a.w) * __uint_as_float(b.w)));
    }
    __device__ static __forceinline__ uint4 add(const uint4 &a, const uint4 &b) {
        return make_uint4(__float_as_uint(__uint_as_float(a.x) + __uint_as_float(b.x)),
                          __float_as_uint(__uint_as_float(a.y) + __uint_as_float(b.y)),
                          __float_as_uint(__uint_as_float(a.z) + __uint_as_float(b.z)),
                          __float_as_uint(__uint_as_float(a.w) + __uint_as_float(b.w)));
    }
    using AbsMax = float;
    __device__ static __forceinline__ AbsMax absmax_init() { return 0.f; }
    __device__ static __forceinline__ void absmax_update(AbsMax &m, const uint4 &a) {
        m = fmaxf(fmaxf(m, fabsf(__uint_as_float(a.x))), fabsf(__uint_as_float(a.y)));
        m = fmaxf(fmaxf(m, fabsf(__uint_as_float(a.z))), fabsf(__uint_as_float(a.w)));
    }
    __device__ static __forceinline__ float absmax_value(AbsMax m) { return m; }
};

// ---------------------------------------------------------------------------------------
// reductions: xor-shuffle inside a warp, one shared-memory hop across warps.  Every thread
// of the block must call these (threads without data pass the identity).  `sm` holds 32
// floats and must not be reused by another reduction before the next block-wide barrier.
// ---------------------------------------------------------------------------------------
__device__ __forceinline__ float warp_sum(float v) {
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
    return v;
}
__device__ __forceinline__ float warp_max(float v) {
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) v = fmaxf(v, __shfl_xor_sync(0xffffffffu, v, o));
    return v;
}
// A group of warps that reduces together: the whole CTA (bar 0), or one role of a kernel whose
// warps are specialised (its own named barrier).  `n` is a multiple of 32.
struct Group {
    int tid;   // this thread's index inside the group
    int n;     // threads in the group
    int bar;   // hardware barrier the group synchronises on
};
__device__ __forceinline__ Group whole_cta() { return Group{static_cast<int>(threadIdx.x), static_cast<int>(blockDim.x), 0}; }
__device__ __forceinline__ void group_sync(const Group &g) {
    asm volatile("bar.sync %0, %1;" ::"r"(g.bar), "r"(g.n) : "memory");
}
// After the barrier every thread reads all per-warp partials with broadcast 16-byte loads and
// combines them in warp order (same order in every thread, so the result is uniform).
__device__ __forceinline__ float block_sum(float v, float *sm, const Group &g) {
    const int lane = g.tid & 31, warp = g.tid >> 5, nwarps = g.n >> 5;
    v = warp_sum(v);
    if (nwarps == 1) return v;
    if (lane == 0) sm[warp] = v;
    if (warp == 0 && lane >= nwarps) sm[lane] = 0.f;   // pad to a multiple of four
    group_sync(g);
    float acc = 0.f;
    for (int i = 0; i < nwarps; i += 4) {
        const float4 q = *reinterpret_cast<const float4 *>(sm + i);
        acc += (q.x + q.y) + (q.z + q.w);
    }
    return acc;
}
__device__ __forceinline__ float block_max(float v, float *sm, const Group &g) {
    const int lane = g.tid & 31, warp = g.tid >> 5, nwarps = g.n >> 5;
    v = warp_max(v);
    if (nwarps == 1) return v;
    if (lane == 0) sm[warp] = v;
    if (warp == 0 && lane >= nwarps) sm[lane] = 0.f;   // operands are magnitudes, so 0 is the identity
    group_sync(g);
    float acc = 0.f;
    for (int i = 0; i < nwarps; i += 4) {
        const float4 q = *reinterpret_cast<const float4 *>(sm + i);
        acc = fmaxf(fmaxf(acc, fmaxf(q.x, q.y)), fmaxf(q.z, q.w));
    }
    return acc;
}

// ---------------------------------------------------------------------------------------
// programmatic dependent launch: the first statement of every kernel that is launched with
// the programmatic-serialization attribute.  Waits until the preceding grid of the stream has
// completed and its writes are visible (a no-op in an ordinary launch), then lets the grid
// that follows begin to place its CTAs, which will wait here in their turn.
// ---------------------------------------------------------------------------------------
__device__ __forceinline__ void grid_dependency_sync() {
    asm volatile("griddepcontrol.wait;" ::: "memory");
    asm volatile("griddepcontrol.launch_dependents;" ::: "memory");
}

// ---------------------------------------------------------------------------------------
// bulk copies (the TMA unit without a tensor map): whole rows travel from global to shared
// memory asynchronously and announce their arrival on an mbarrier, so a CTA keeps loads in
// flight while it computes.  Source, destination and size must be multiples of 16 bytes.
// ---------------------------------------------------------------------------------------
__device__ __forceinline__ uint32_t smem_addr(const void *p) { return static_cast<uint32_t>(__cvta_generic_to_shared(p)); }
__device__ __forceinline__ void mbar_init(uint64_t *bar, int arrivals) {
    asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(smem_addr(bar)), "r"(arrivals) : "memory");
}
// Makes freshly initialised mbarriers visible to the bulk-copy unit (follow with a block barrier).
__device__ __forceinline__ void mbar_init_fence() { asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory"); }
__device__ __forceinline__ void mbar_expect_bytes(uint64_t *bar, uint32_t bytes) {
    asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(smem_addr(bar)), "r"(bytes) : "memory");
}
__device__ __forceinline__ void bulk_load(void *smem_dst, const void *global_src, uint32_t bytes, uint64_t *bar) {
    asm volatile("cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];"
                 ::"r"(smem_addr(smem_dst)), "l"(global_src), "r"(bytes), "r"(smem_addr(bar)) : "memory");
}
// Waits for the phase of `bar` with the given parity to complete.  The copies it waits for are
// this CTA's own and always complete; the loop is bounded all the same and returns false when
// it gives up.
__device__ __forceinline__ bool mbar_wait(uint64_t *bar, uint32_t parity) {
    const uint32_t a = smem_addr(bar);
    for (uint32_t spin = 0; spin < (1u << 24); ++spin) {
        uint32_t ok;
        asm volatile("{\n\t.reg .pred p;\n\tmbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n\tselp.u32 %0, 1, 0, p;\n\t}"
                     : "=r"(ok) : "r"(a), "r"(parity) : "memory");
        if (ok) return true;
    }
    return false;
}

// ---------------------------------------------------------------------------------------
// thread-block clusters: a row may be split over the CTAs of a cluster, which then combine
// their partial reductions through distributed shared memory.  In a launch without a cluster
// attribute the cluster is the CTA itself (size 1, rank 0).
// ---------------------------------------------------------------------------------------
__device__ __forceinline__ int cluster_cta_rank() {
    uint32_t r;
    asm volatile("mov.u32 %0, %%cluster_ctarank;" : "=r"(r));
    return static_cast<int>(r);
}
__device__ __forceinline__ int cluster_size() {
    uint32_t n;
    asm volatile("mov.u32 %0, %%cluster_nctarank;" : "=r"(n));
    return static_cast<int>(n);
}
// Barrier over all threads of the cluster; shared-memory writes made before it (local or to
// another CTA of the cluster) are visible to every thread of the cluster after it.
__device__ __forceinline__ void cluster_barrier() {
    asm volatile("barrier.cluster.arrive.release.aligned;\n\tbarrier.cluster.wait.acquire.aligned;" ::: "memory");
}
// Stores `v` at the address `local` names, but in the shared memory of CTA `cta` of this cluster.
__device__ __forceinline__ void st_cluster_f32(float *local, int cta, float v) {
    const uint32_t a = static_cast<uint32_t>(__cvta_generic_to_shared(local));
    uint32_t remote;
    asm volatile("mapa.shared::cluster.u32 %0, %1, %2;" : "=r"(remote) : "r"(a), "r"(cta));
    asm volatile("st.shared::cluster.f32 [%0], %1;" ::"r"(remote), "f"(v) : "memory");
}
// Every CTA of the cluster passes its own value (uniform across its threads); returns, in every
// thread of every CTA, the combination of all of them taken in CTA order.  `slots` is this
// CTA's array of 8 floats; it may be reused after the next cluster_barrier but one.
template <bool MAX>
__device__ __forceinline__ float cluster_combine(float v, float *slots, int cl_rank, int cl_size) {
    if (cl_size == 1) return v;
    if (threadIdx.x < cl_size) st_cluster_f32(slots + cl_rank, threadIdx.x, v);   // clusters only occur with whole-CTA groups
    cluster_barrier();
    float acc = slots[0];
    for (int i = 1; i < cl_size; ++i) acc = MAX ? fmaxf(acc, slots[i]) : acc + slots[i];
    return acc;
}

// ---------------------------------------------------------------------------------------
// fp32 -> FP8 e4m3, round to nearest even, saturating: one hardware instruction per pair
// ---------------------------------------------------------------------------------------
__device__ __forceinline__ uint32_t cvt_e4m3x2(float lo, float hi) {
    uint16_t r;
    asm("cvt.rn.satfinite.e4m3x2.f32 %0, %1, %2;" : "=h"(r) : "f"(hi), "f"(lo));
    return r;
}
// Two fp32 pairs (elements e, e+1 and e+2, e+3) -> four FP8 e4m3fn bytes in element order.
__device__ __forceinline__ uint32_t cvt_e4m3x4_pairs(f32x2 a, f32x2 b) {
    uint32_t w;
    asm("{\n\t.reg .b16 lo, hi;\n\t.reg .f32 a0, a1, b0, b1;\n\t"
        "mov.b64 {a0, a1}, %1;\n\tmov.b64 {b0, b1}, %2;\n\t"
        "cvt.rn.satfinite.e4m3x2.f32 lo, a1, a0;\n\tcvt.rn.satfinite.e4m3x2.f32 hi, b1, b0;\n\t"
        "mov.b32 %0, {lo, hi};\n\t}"
        : "=r"(w) : "l"(a), "l"(b));
    return w;
}
// A byte equal to 0x80 (negative zero in e4m3fn, NaN in e4m3fnuz) becomes 0x00; others unchanged.
__device__ __forceinline__ uint32_t fold_negative_zero_bytes(uint32_t w) {
    const uint32_t low7 = w & 0x7f7f7f7fu;
    const uint32_t nonzero7 = (low7 + 0x7f7f7f7fu) & 0x80808080u;   // bit 7 set where low 7 bits != 0
    return low7 | (w & nonzero7);
}
// Four floats -> four FP8 bytes (little-endian lane order).  For the fnuz flavour the value
// is doubled (e4m3fnuz has exponent bias 8 where e4m3fn has 7, so code_fnuz(x) == code_fn(2x))
// and the negative-zero pattern 0x80, which fnuz reads as NaN, is folded to +0.
__device__ __forceinline__ uint32_t cvt_e4m3x4(float a, float b, float c, float d, int fnuz) {
    if (fnuz) {
        a += a; b += b; c += c; d += d;
    }
    uint32_t w = cvt_e4m3x2(a, b) | (cvt_e4m3x2(c, d) << 16);
    if (fnuz) {
        // a byte equal to 0x80 becomes 0x00; every other byte is unchanged
        uint32_t low7 = w & 0x7f7f7f7fu;
        uint32_t nonzero7 = (low7 + 0x7f7f7f7fu) & 0x80808080u;   // bit 7 set where low 7 bits != 0
        w = low7 | (w & nonzero7);
    }
    return w;
}

// ---------------------------------------------------------------------------------------
// cross-GPU hand-off without flags or fences: the data announces itself
// ---------------------------------------------------------------------------------------
// Staging memory rests in a known state: every 32-bit word holds kEmptyWord.  A producer
// (a peer GPU, or another CTA of this GPU) overwrites whole 16-byte vectors with payload that
// never contains that word; the consumer polls the vector until none of its four words is
// kEmptyWord (aligned 32-bit stores are indivisible, so no ordering between the words or
// between vectors is needed), uses it, and writes kEmptyWord back so the location is at rest
// for its next use.  Nothing is fenced and nothing is signalled: NVLink carries only the
// payload, and a consumer starts the moment its own 16 bytes have landed.
//
// kEmptyWord is two negative zeros in the 16-bit formats.  A payload word equal to it is
// rewritten before it is sent: to two positive zeros for 16-bit types (the sum of partials is
// unchanged unless every rank contributes -0) and to the neighbouring denormal for fp32.
//
// Replaces the counter barrier of src/common/communicator.h:79-113 (st_flag / ld_flag / sync).
constexpr uint32_t kEmptyWord = 0x80008000u;

template <typename T>
__device__ __forceinline__ uint4 payload(uint4 v) {
    constexpr uint32_t repl = sizeof(T) == 4 ? 0x80008001u : 0u;
    v.x = v.x == kEmptyWord ? repl : v.x;
    v.y = v.y == kEmptyWord ? repl : v.y;
    v.z = v.z == kEmptyWord ? repl : v.z;
    v.w = v.w == kEmptyWord ? repl : v.w;
    return v;
}
__device__ __forceinline__ bool landed(const uint4 &v) {
    return v.x != kEmptyWord && v.y != kEmptyWord && v.z != kEmptyWord && v.w != kEmptyWord;
}
// Read of staging memory that another GPU (or CTA) is writing: always served by L2.
__device__ __forceinline__ uint4 ld_poll(const void *p) {
    uint4 v;
    asm volatile("ld.volatile.global.v4.u32 {%0, %1, %2, %3}, [%4];"
                 : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w) : "l"(p) : "memory");
    return v;
}
__device__ __forceinline__ void st_empty(void *p) {
    *reinterpret_cast<uint4 *>(p) = make_uint4(kEmptyWord, kEmptyWord, kEmptyWord, kEmptyWord);
}
__device__ __forceinline__ uint32_t ld_volatile_u32(const uint32_t *addr) {
    uint32_t v;
    asm volatile("ld.volatile.global.u32 %0, [%1];" : "=r"(v) : "l"(addr) : "memory");
    return v;
}
__device__ __forceinline__ unsigned long long global_timer_ns() {
    unsigned long long t;
    asm volatile("mov.u64 %0, %%globaltimer;" : "=l"(t));
    return t;
}

// ---------------------------------------------------------------------------------------
// exchange through symmetric memory: NVSwitch multicast (multimem) and 64-bit flags
// ---------------------------------------------------------------------------------------
// A multicast address names the same offset in every rank's symmetric buffer.  A multimem load
// with reduction returns the sum of that location over all ranks, added up inside the switch
// (fp32 accumulation for the 16-bit types, one rounding); a multimem store writes all ranks.
template <typename T>
__device__ __forceinline__ uint4 multimem_ld_sum(const void *mc);
template <>
__device__ __forceinline__ uint4 multimem_ld_sum<__nv_bfloat16>(const void *mc) {
    uint4 v;
    asm volatile("multimem.ld_reduce.relaxed.sys.global.add.acc::f32.v4.bf16x2 {%0, %1, %2, %3}, [%4];"
                 : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w) : "l"(mc) : "memory");
    return v;
}
template <>
__device__ __forceinline__ uint4 multimem_ld_sum<__half>(const void *mc) {
    uint4 v;
    asm volatile("multimem.ld_reduce.relaxed.sys.global.add.acc::f32.v4.f16x2 {%0, %1, %2, %3}, [%4];"
                 : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w) : "l"(mc) : "memory");
    return v;
}
template <>
__device__ __forceinline__ uint4 multimem_ld_sum<float>(const void *mc) {
    uint4 v;
    asm volatile("multimem.ld_reduce.relaxed.sys.global.add.v4.f32 {%0, %1, %2, %3}, [%4];"
                 : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w) : "l"(mc) : "memory");
    return v;
}
__device__ __forceinline__ void multimem_st(void *mc, const uint4 &v) {
    asm volatile("multimem.st.relaxed.sys.global.v4.f32 [%0], {%1, %2, %3, %4};"
                 ::"l"(mc), "r"(v.x), "r"(v.y), "r"(v.z), "r"(v.w) : "memory");
}
// Flag stores with release semantics (after a block barrier and a system fence they publish the
// CTA's earlier writes), to one rank or through the multicast address to all of them.
__device__ __forceinline__ void st_flag_release(unsigned long long *p, unsigned long long v) {
    asm volatile("st.release.sys.global.u64 [%0], %1;" ::"l"(p), "l"(v) : "memory");
}
__device__ __forceinline__ void multimem_st_flag_release(unsigned long long *mc, unsigned long long v) {
    asm volatile("multimem.st.release.sys.global.u64 [%0], %1;" ::"l"(mc), "l"(v) : "memory");
}
__device__ __forceinline__ unsigned long long ld_flag_acquire(const unsigned long long *p) {
    unsigned long long v;
    asm volatile("ld.acquire.sys.global.u64 %0, [%1];" : "=l"(v) : "l"(p) : "memory");
    return v;
}

constexpr uint32_t kSpinCap = 1u << 24;   // hard bound on polls of one wait, independent of the timer

__device__ __forceinline__ void record_status(LocalState *st, uint32_t code, int rank, int block, int stage,
                                              int peer, uint32_t word) {
    if (atomicCAS(&st->status[0], 0u, code) == 0u) {
        st->status[1] = rank;
        st->status[2] = block;
        st->status[3] = stage;
        st->status[4] = peer;
        st->status[5] = threadIdx.x;
        st->status[6] = word;
    }
    atomicExch(&st->abort, 1u);
}

// `v` is the first read of the vector at `addr`.  Polls until the vector has landed, within the
// workspace's time budget (and kSpinCap polls); on expiry records where it gave up, latches
// `abort` so that later waits return at once, and hands back whatever is there: the kernel
// always terminates.
static __device__ __noinline__ uint4 wait_landed_slow(const void *addr, uint4 v, LocalState *st, int rank, int stage, int peer) {
    unsigned long long t0 = 0;
    for (uint32_t it = 1; it <= kSpinCap; ++it) {
        __nanosleep(40);
        v = ld_poll(addr);
        if (landed(v)) return v;
        if ((it & 63u) == 0u) {
            const unsigned long long now = global_timer_ns();
            if (t0 == 0) {
                t0 = now;
                if (ld_volatile_u32(&st->abort)) return v;
            } else if (now - t0 > st->timeout_ns || ld_volatile_u32(&st->abort)) {
                record_status(st, kStatusWaitTimeout, rank, blockIdx.x, stage, peer, v.x);
                return v;
            }
        }
    }
    record_status(st, kStatusSpinCap, rank, blockIdx.x, stage, peer, v.x);
    return v;
}
__device__ __forceinline__ uint4 wait_landed(const void *addr, uint4 v, LocalState *st, int rank, int stage, int peer) {
    return landed(v) ? v : wait_landed_slow(addr, v, st, rank, stage, peer);
}

// Row-block ready words of the local input: a producer on this GPU (the GEMM that writes the partial sums,
// or a copy engine) stores `want` (or more) into a word after the rows it stands for are complete; the
// acquire load orders this thread's later reads of those rows behind it.  Same bounds and reporting as
// wait_landed; `peer` is this rank itself.  Returns false when it gave up.
static __device__ __noinline__ bool wait_ready_slow(const uint32_t *word, uint32_t want, LocalState *st, int rank) {
    unsigned long long t0 = 0;
    for (uint32_t it = 0; it <= kSpinCap; ++it) {
        uint32_t seen;
        asm volatile("ld.acquire.gpu.global.u32 %0, [%1];" : "=r"(seen) : "l"(word) : "memory");
        if (seen >= want) return true;
        if ((it & 63u) == 63u) {
            const unsigned long long now = global_timer_ns();
            if (t0 == 0) {
                t0 = now;
                if (ld_volatile_u32(&st->abort)) return false;
            } else if (now - t0 > st->timeout_ns || ld_volatile_u32(&st->abort)) {
                record_status(st, kStatusWaitTimeout, rank, blockIdx.x, kStageReady, rank, seen);
                return false;
            }
        }
        __nanosleep(100);
    }
    record_status(st, kStatusSpinCap, rank, blockIdx.x, kStageReady, rank, 0u);
    return false;
}
__device__ __forceinline__ bool wait_ready(const uint32_t *word, uint32_t want, LocalState *st, int rank) {
    uint32_t seen;
    asm volatile("ld.acquire.gpu.global.u32 %0, [%1];" : "=r"(seen) : "l"(word) : "memory");
    return seen >= want ? true : wait_ready_slow(word, want, st, rank);
}

// Polls a flag until it has reached `want` (flags only grow), with the same bounds and the same
// reporting as wait_landed.  Returns false when it gave up.
static __device__ __noinline__ bool wait_flag(const unsigned long long *flag, unsigned long long want, LocalState *st, int rank,
                                              int stage, int peer) {
    unsigned long long t0 = 0;
    for (uint32_t it = 0; it <= kSpinCap; ++it) {
        const unsigned long long seen = ld_flag_acquire(flag);
        if (seen >= want) return true;
        if ((it & 63u) == 63u) {
            const unsigned long long now = global_timer_ns();
            if (t0 == 0) {
                t0 = now;
                if (ld_volatile_u32(&st->abort)) return false;
            } else if (now - t0 > st->timeout_ns || ld_volatile_u32(&st->abort)) {
                record_status(st, kStatusWaitTimeout, rank, blockIdx.x, stage, peer, static_cast<uint32_t>(seen));
                return false;
            }
        }
        __nanosleep(20);
    }
    record_status(st, kStatusSpinCap, rank, blockIdx.x, stage, peer, 0u);
    return false;
}

}  // namespace gpuk

// The consumer of the fused operator's FP8 output: y = (x_fp8 . w_fp8^T) * x_scale[token] * w_scale[channel]
// for a handful of tokens (decode), i.e. the linear layer that follows the norm in a tensor-parallel
// block (F.linear in model/tensor_parallel.py:66 of the reference, which has no FP8 path of its own).
//
// With at most 32 tokens the product is a weight-streaming problem: every weight byte is read once
// and used for 32 multiply-adds, so the kernel is bound by HBM, not by the tensor pipe.  That decides
// the design:
//
//   * weights [n, k] (k contiguous, e4m3) are the 16-row operand of the warp-level mma and the
//     activations [tokens, k] its 8-column operand, so one weight fragment is used for all four
//     groups of 8 tokens; the weights go from global memory straight into the fragment registers.
//     sm_100 has no native FP8 path for mma.sync (ptxas expands an e4m3 mma into conversions and
//     f16 HMMAs per instruction, 170 instructions per 64-byte k step as first written), so the
//     kernel converts e4m3 -> f16 itself (exact), once per weight fragment instead of once per
//     token group, and issues mma.sync.m16n8k16.f16.f16.f32.  Products of two e4m3 values are exact
//     in the fp32 accumulator either way.
//   * fragment loads are 16 bytes per thread.  The instruction wants thread (g, t) of a warp to hold
//     k = 2t, 2t+1 and 2t+8, 2t+9 of row g; a dot product does not care about the order of k as
//     long as both operands use the same order, so thread (g, t) instead loads the 16 contiguous
//     bytes k0 + 16t .. k0 + 16t + 15 of its row -- of the weights and of the activations alike --
//     and feeds them to four consecutive mma instructions.  A warp's load then covers 64 contiguous
//     bytes of 8 rows: whole 32-byte sectors, nothing wasted.
//   * a tile of 128 output channels is shared by a thread-block cluster of KS CTAs that split k;
//     inside a CTA the eight warps split the channels (16 each, one fragment), so a CTA needs no
//     reduction of its own.  The activations of the CTA's k-range are staged through shared memory once (cp.async)
//     and read by all four warps.  The KS partial tiles are summed through distributed shared
//     memory in a fixed order (deterministic, no atomics), scaled, rounded once and stored.
//
// Activation traffic is (n / 128) x tokens x k bytes out of L2 against n x k bytes of weights from
// HBM: a quarter of it at 32 tokens.
#include <cuda_bf16.h>
#include <cuda_runtime.h>

#include <cstdint>

#include "../../include/gpuk_b200.h"
#include "launch.cuh"

namespace gpuk {
namespace {

constexpr int kTileN = 128;        // output channels per cluster
constexpr int kWarps = 8;          // per CTA; each owns kTileN / kWarps = 16 channels = one 16-row fragment
constexpr int kRing = 8;           // k steps of weights a thread keeps in flight: 16 x 16 bytes
constexpr int kTokens = 32;        // token capacity of one pass: four groups of 8
constexpr int kStepBytes = 64;     // k bytes one warp-wide 16-byte load covers per row
constexpr int kChunkSteps = 16;    // k steps staged per round: 1 KiB of every token's row
constexpr int kXRow = kChunkSteps * kStepBytes + 64;   // shared-memory row pitch; 64 mod 128 keeps 16-byte reads conflict-free
constexpr int kPartPitch = 36;     // floats per channel row of the partial tile (32 tokens + padding)

struct Fp8LinearParams {
    const uint8_t *x;        // [m, k] e4m3
    const float *x_scale;    // [m]
    const uint8_t *w;        // [n, k] e4m3
    const float *w_scale;    // [n]
    __nv_bfloat16 *out;      // [m, n]
    int m, n, k;
    int ks;                  // CTAs per cluster = parts k is split into (planned; checked in the kernel)
    int packed;              // weight layout: 0 = [n, k] row-major, 1 = blocked (gpuk_fp8_pack_weight)
    int *status;             // set to 1 when the launch did not carry the planned cluster (nothing is written then)
};

__device__ __forceinline__ uint4 ld_weights(const uint8_t *p) {
    uint4 v;
    asm volatile("ld.global.nc.L1::no_allocate.L2::128B.v4.u32 {%0, %1, %2, %3}, [%4];"
                 : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w) : "l"(p));
    return v;
}

__device__ __forceinline__ void cp_async16(void *smem, const void *gmem, bool valid) {
    const uint32_t s = static_cast<uint32_t>(__cvta_generic_to_shared(smem));
    const int bytes = valid ? 16 : 0;     // 0: the 16 bytes are filled with zeros
    asm volatile("cp.async.cg.shared.global [%0], [%1], 16, %2;" ::"r"(s), "l"(gmem), "r"(bytes) : "memory");
}

// Four e4m3 values in a 32-bit register -> two registers of two f16 each (exact: every e4m3 value is an f16 value).
__device__ __forceinline__ void e4m3x4_to_f16x4(uint32_t v, uint32_t &lo, uint32_t &hi) {
    asm("{\n\t.reg .b16 a, b;\n\tmov.b32 {a, b}, %2;\n\tcvt.rn.f16x2.e4m3x2 %0, a;\n\tcvt.rn.f16x2.e4m3x2 %1, b;\n\t}"
        : "=r"(lo), "=r"(hi) : "r"(v));
}
// 16 e4m3 bytes -> 8 registers of f16 pairs, in byte order
__device__ __forceinline__ void e4m3x16_to_f16(const uint4 &v, uint32_t (&h)[8]) {
    e4m3x4_to_f16x4(v.x, h[0], h[1]);
    e4m3x4_to_f16x4(v.y, h[2], h[3]);
    e4m3x4_to_f16x4(v.z, h[4], h[5]);
    e4m3x4_to_f16x4(v.w, h[6], h[7]);
}

__device__ __forceinline__ void mma_f16(float (&d)[4], uint32_t a0, uint32_t a1, uint32_t a2, uint32_t a3, uint32_t b0, uint32_t b1) {
    asm volatile("mma.sync.aligned.m16n8k16.row.col.f32.f16.f16.f32 {%0, %1, %2, %3}, {%4, %5, %6, %7}, {%8, %9}, {%0, %1, %2, %3};"
                 : "+f"(d[0]), "+f"(d[1]), "+f"(d[2]), "+f"(d[3])
                 : "r"(a0), "r"(a1), "r"(a2), "r"(a3), "r"(b0), "r"(b1));
}

__device__ __forceinline__ float ld_cluster_f32(const float *local, int cta) {
    const uint32_t a = static_cast<uint32_t>(__cvta_generic_to_shared(local));
    uint32_t remote;
    float v;
    asm volatile("mapa.shared::cluster.u32 %0, %1, %2;" : "=r"(remote) : "r"(a), "r"(cta));
    asm volatile("ld.shared::cluster.f32 %0, [%1];" : "=f"(v) : "r"(remote) : "memory");
    return v;
}

__global__ void __launch_bounds__(kWarps * 32, 2) fp8_linear_skinny_kernel(const __grid_constant__ Fp8LinearParams p) {
    // activations of one round (32 tokens x 1 KiB); afterwards the CTA's partial tile (128 x 32 fp32) lives in the same memory
    __shared__ __align__(16) unsigned char smem[kTokens * kXRow];
    static_assert(kTileN * kPartPitch * 4 <= kTokens * kXRow, "the partial tile reuses the activation stage");
    static_assert(kChunkSteps % kRing == 0, "a round of activations is a whole number of ring turns");
    grid_dependency_sync();
    const int ks = cluster_size(), part = cluster_cta_rank();
    if (ks != p.ks) {
        if (threadIdx.x == 0) *p.status = 1;
        return;
    }
    const int tile = blockIdx.x / ks;
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31, g = lane >> 2, t = lane & 3;
    const int n0 = tile * kTileN + warp * 16;
    // this CTA's share of the k steps: contiguous, the first `extra` parts take one step more
    const int steps = p.k / kStepBytes;
    const int base = steps / ks, extra = steps % ks;
    const int s_begin = part * base + (part < extra ? part : extra);
    const int s_end = s_begin + base + (part < extra ? 1 : 0);

    const int qn = (p.m + 7) / 8;      // groups of 8 tokens in use
    float acc[4][4];
#pragma unroll
    for (int q = 0; q < 4; ++q)
#pragma unroll
        for (int e = 0; e < 4; ++e) acc[q][e] = 0.f;

    // the two weight rows this thread reads: rows g and g + 8 of the warp's fragment
    // Row-major weights: a k step of the warp's fragment is 64 bytes of 16 rows that lie k bytes apart.  Blocked
    // weights: the same 16 x 64 bytes are one contiguous KiB (row r of the fragment at r * 64) and consecutive k steps
    // follow each other, so a warp streams its fragment's rows as one sequential run of memory.
    const size_t step_stride = p.packed ? 16 * kStepBytes : kStepBytes;
    const uint8_t *wrow0 = p.packed ? p.w + static_cast<size_t>(n0 / 16) * p.k * 16 + g * kStepBytes + 16 * t
                                    : p.w + static_cast<size_t>(n0 + g) * p.k + 16 * t;
    const uint8_t *wrow1 = wrow0 + (p.packed ? static_cast<size_t>(8) * kStepBytes : static_cast<size_t>(8) * p.k);

    // Weights travel through a ring of eight k steps held in registers: a slot is refilled with the step eight ahead
    // as soon as it has been multiplied, so up to 256 bytes per thread (64 KiB per CTA) are in flight at any time.
    uint4 ring[kRing][2];
#pragma unroll
    for (int u = 0; u < kRing; ++u)
        if (s_begin + u < s_end) {
            ring[u][0] = ld_weights(wrow0 + static_cast<size_t>(s_begin + u) * step_stride);
            ring[u][1] = ld_weights(wrow1 + static_cast<size_t>(s_begin + u) * step_stride);
        }
    for (int s = s_begin; s < s_end; s += kRing) {
        const int in_chunk = (s - s_begin) % kChunkSteps;
        if (in_chunk == 0) {
            // stage the activations of the next 16 k steps (all warps read all of them)
            const int nsteps = s_end - s < kChunkSteps ? s_end - s : kChunkSteps;
            __syncthreads();      // everyone is done with the previous round's activations
            const int row_chunks = nsteps * (kStepBytes / 16);
            for (int i = threadIdx.x; i < qn * 8 * row_chunks; i += blockDim.x) {
                const int tok = i / row_chunks, c = i - tok * row_chunks;
                cp_async16(smem + tok * kXRow + c * 16, p.x + static_cast<size_t>(tok < p.m ? tok : 0) * p.k + static_cast<size_t>(s) * kStepBytes + c * 16,
                           tok < p.m);
            }
            asm volatile("cp.async.commit_group;\n\tcp.async.wait_group 0;" ::: "memory");
            __syncthreads();
        }
#pragma unroll
        for (int u = 0; u < kRing; ++u) {
            const int st = s + u;
            if (st < s_end) {
                // the weights are converted once and used for every token group
                uint32_t w0[8], w1[8];
                e4m3x16_to_f16(ring[u][0], w0);
                e4m3x16_to_f16(ring[u][1], w1);
#pragma unroll
                for (int q = 0; q < 4; ++q) {
                    if (q < qn) {      // token groups that hold no token are skipped (uniform across the CTA)
                        const uint4 xf = *reinterpret_cast<const uint4 *>(smem + (q * 8 + g) * kXRow + (in_chunk + u) * kStepBytes + 16 * t);
                        uint32_t xh[8];
                        e4m3x16_to_f16(xf, xh);
#pragma unroll
                        for (int i = 0; i < 4; ++i) mma_f16(acc[q], w0[2 * i], w1[2 * i], w0[2 * i + 1], w1[2 * i + 1], xh[2 * i], xh[2 * i + 1]);
                    }
                }
                if (st + kRing < s_end) {
                    ring[u][0] = ld_weights(wrow0 + static_cast<size_t>(st + kRing) * step_stride);
                    ring[u][1] = ld_weights(wrow1 + static_cast<size_t>(st + kRing) * step_stride);
                }
            }
        }
    }

    // this CTA's partial tile: channel-major, fp32
    __syncthreads();
    float *partial = reinterpret_cast<float *>(smem);
#pragma unroll
    for (int q = 0; q < 4; ++q) {
        const int ch = warp * 16 + g, tok = q * 8 + 2 * t;
        *reinterpret_cast<float2 *>(partial + ch * kPartPitch + tok) = make_float2(acc[q][0], acc[q][1]);
        *reinterpret_cast<float2 *>(partial + (ch + 8) * kPartPitch + tok) = make_float2(acc[q][2], acc[q][3]);
    }
    cluster_barrier();
    // CTA `part` finishes channels [part * per, part * per + per) of the tile: sum over the cluster in CTA order
    const int per = kTileN / ks;
    for (int e = threadIdx.x; e < per * kTokens; e += blockDim.x) {
        const int ch = part * per + e % per, tok = e / per;
        float sum = 0.f;
        for (int c = 0; c < ks; ++c) sum += ld_cluster_f32(partial + ch * kPartPitch + tok, c);
        const int n = tile * kTileN + ch;
        if (tok < p.m) p.out[static_cast<size_t>(tok) * p.n + n] = __float2bfloat16_rn(sum * p.x_scale[tok] * p.w_scale[n]);
    }
    cluster_barrier();     // nobody leaves while its partial tile may still be read
}

__global__ void clear_status_kernel(int *status) { *status = 0; }

// [n, k] row-major -> blocked: block (n / 16, k / 64) holds 16 rows x 64 bytes, row r at r * 64; blocks of one
// 16-row band follow each other along k.  One 16-byte vector per thread.
__global__ void pack_weight_kernel(const uint4 *w, uint4 *packed, int n, int k) {
    const size_t vecs = static_cast<size_t>(n) * k / 16;
    const int kv = k / 16;      // vectors per row
    for (size_t i = blockIdx.x * static_cast<size_t>(blockDim.x) + threadIdx.x; i < vecs; i += static_cast<size_t>(gridDim.x) * blockDim.x) {
        const int row = static_cast<int>(i / kv), v = static_cast<int>(i % kv);
        const size_t dst = (static_cast<size_t>(row / 16) * (k / kStepBytes) + v / 4) * 64 + (row % 16) * 4 + v % 4;
        packed[dst] = w[i];
    }
}

int *g_status_by_device[64] = {};   // one device word per GPU, allocated by the first call on it

}  // namespace
}  // namespace gpuk

using namespace gpuk;

extern "C" int gpuk_fp8_linear_skinny(const void *x_fp8, const float *x_scale, const void *w_fp8, const float *w_scale,
                                      void *out_bf16, int m, int n, int k, int w_layout, int k_split, void *stream) {
    if (!x_fp8 || !x_scale || !w_fp8 || !w_scale || !out_bf16) return set_last_error(GPUK_ERR_INVALID_ARGUMENT, "fp8_linear: null pointer");
    if (m < 0 || n <= 0 || k <= 0) return set_last_error(GPUK_ERR_INVALID_ARGUMENT, "fp8_linear: bad shape %d x %d x %d", m, n, k);
    if (m == 0) return GPUK_OK;
    if (m > kTokens) return set_last_error(GPUK_ERR_UNSUPPORTED, "fp8_linear: %d tokens; this kernel is built for at most %d (use a library GEMM beyond)", m, kTokens);
    if (n % kTileN || k % kStepBytes)
        return set_last_error(GPUK_ERR_UNSUPPORTED, "fp8_linear: n must be a multiple of %d and k of %d (got %d, %d)", kTileN, kStepBytes, n, k);
    if ((reinterpret_cast<uintptr_t>(x_fp8) | reinterpret_cast<uintptr_t>(w_fp8)) & 15u)
        return set_last_error(GPUK_ERR_INVALID_ARGUMENT, "fp8_linear: operands must be 16-byte aligned");
    if (w_layout != 0 && w_layout != 1) return set_last_error(GPUK_ERR_INVALID_ARGUMENT, "fp8_linear: w_layout must be 0 (row-major) or 1 (blocked)");
    if (k_split != 0 && k_split != 1 && k_split != 2 && k_split != 4 && k_split != 8)
        return set_last_error(GPUK_ERR_INVALID_ARGUMENT, "fp8_linear: k_split must be 0, 1, 2, 4 or 8");
    int device = 0, sms = 148;
    if (cudaGetDevice(&device) != cudaSuccess) return set_last_error(GPUK_ERR_CUDA, "fp8_linear: no current device");
    cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, device);
    // split k as far as the whole grid still runs as one wave (two CTAs per SM) and every part keeps a few steps
    int ks = k_split;
    if (ks == 0) {
        ks = 1;
        while (ks < 8 && (n / kTileN) * ks * 2 <= 2 * sms && k / kStepBytes >= 8 * ks) ks *= 2;
    }
    int **status_by_device = g_status_by_device;
    if (device < 0 || device >= 64) return set_last_error(GPUK_ERR_UNSUPPORTED, "fp8_linear: device index %d", device);
    if (!status_by_device[device]) {
        int *s = nullptr;
        if (cudaMalloc(&s, sizeof(int)) != cudaSuccess) return set_last_error(GPUK_ERR_CUDA, "fp8_linear: cannot allocate the status word");
        clear_status_kernel<<<1, 1, 0, static_cast<cudaStream_t>(stream)>>>(s);
        status_by_device[device] = s;
    }
    Fp8LinearParams p = {static_cast<const uint8_t *>(x_fp8), x_scale, static_cast<const uint8_t *>(w_fp8), w_scale,
                         static_cast<__nv_bfloat16 *>(out_bf16), m, n, k, ks, w_layout, status_by_device[device]};
    void *args[] = {&p};
    cudaError_t e = launch_kernel(reinterpret_cast<const void *>(&fp8_linear_skinny_kernel), (n / kTileN) * ks, kWarps * 32, ks, false, args,
                                  static_cast<cudaStream_t>(stream));
    if (e != cudaSuccess) return set_last_error(GPUK_ERR_CUDA, "fp8_linear: launch failed: %s", cudaGetErrorString(e));
    return GPUK_OK;
}

extern "C" int gpuk_fp8_pack_weight(const void *w_fp8, void *packed, int n, int k, void *stream) {
    if (!w_fp8 || !packed || w_fp8 == packed) return set_last_error(GPUK_ERR_INVALID_ARGUMENT, "fp8_pack_weight: null or aliased pointers");
    if (n <= 0 || k <= 0 || n % 16 || k % kStepBytes)
        return set_last_error(GPUK_ERR_UNSUPPORTED, "fp8_pack_weight: n must be a multiple of 16 and k of %d (got %d, %d)", kStepBytes, n, k);
    if ((reinterpret_cast<uintptr_t>(w_fp8) | reinterpret_cast<uintptr_t>(packed)) & 15u)
        return set_last_error(GPUK_ERR_INVALID_ARGUMENT, "fp8_pack_weight: pointers must be 16-byte aligned");
    pack_weight_kernel<<<1184, 256, 0, static_cast<cudaStream_t>(stream)>>>(static_cast<const uint4 *>(w_fp8), static_cast<uint4 *>(packed), n, k);
    cudaError_t e = cudaGetLastError();
    if (e != cudaSuccess) return set_last_error(GPUK_ERR_CUDA, "fp8_pack_weight: launch failed: %s", cudaGetErrorString(e));
    return GPUK_OK;
}

extern "C" int gpuk_fp8_linear_status(void) {
    int device = 0;
    if (cudaGetDevice(&device) != cudaSuccess || device < 0 || device >= 64) return set_last_error(GPUK_ERR_CUDA, "fp8_linear: no current device");
    if (!g_status_by_device[device]) return GPUK_OK;     // no call on this device yet
    int v = 0;
    if (cudaDeviceSynchronize() != cudaSuccess || cudaMemcpy(&v, g_status_by_device[device], sizeof(v), cudaMemcpyDeviceToHost) != cudaSuccess)
        return set_last_error(GPUK_ERR_CUDA, "fp8_linear: cannot read the status word: %s", cudaGetErrorString(cudaGetLastError()));
    return v ? set_last_error(GPUK_ERR_BAD_LAUNCH, "fp8_linear: a launch ran without its planned thread-block cluster and wrote nothing") : GPUK_OK;
}

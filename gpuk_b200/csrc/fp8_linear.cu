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
//     groups of 8 tokens; every thread fetches exactly the bytes of its own fragment registers.
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
//     reduction of its own.  Weights and activations arrive by cp.async (the pipeline is described at
//     the kernel).  The KS partial tiles are summed through distributed shared memory in a fixed
//     order (deterministic, no atomics), scaled, rounded once and stored.
//
// Activation traffic is (n / 128) x tokens x k bytes out of L2 against n x k bytes of weights from
// HBM: a quarter of it at 32 tokens.
#include <cuda_bf16.h>
#include <cuda_runtime.h>

#include <cstdint>
#include <mutex>

#include "../../include/gpuk_b200.h"
#include "launch.cuh"

namespace gpuk {
namespace {

constexpr int kTileN = 128;        // output channels per cluster
constexpr int kWarps = 8;          // per CTA; each owns kTileN / kWarps = 16 channels = one 16-row fragment
constexpr int kThreads = kWarps * 32;
constexpr int kDepth = 8;          // k steps of weights in flight per thread (cp.async groups): 7 x 32 bytes
constexpr int kTokens = 32;        // token capacity of one pass: four groups of 8
constexpr int kStepBytes = 64;     // k bytes one warp-wide 16-byte load covers per row
constexpr int kXSteps = 8;         // k steps of activations staged together (two such buffers)
constexpr int kXRow = kXSteps * kStepBytes + 64;   // shared-memory row pitch; 64 mod 128 keeps 16-byte reads conflict-free
constexpr int kXBuf = kTokens * kXRow;              // one activation buffer
constexpr int kWSlot = 2 * kThreads * 16;           // one k step of the CTA's weights: two 16-byte vectors per thread
constexpr int kPartPitch = kTileN + 4;              // floats per token row of the partial tile (128 channels + padding)
constexpr int kSmemBytes = kDepth * kWSlot + 2 * kXBuf;   // 64 KiB + 36 KiB: two CTAs per SM
static_assert(kTokens * kPartPitch * 4 <= kDepth * kWSlot, "the partial tile reuses the weight ring");
static_assert((kDepth & (kDepth - 1)) == 0 && kXSteps == kDepth, "slot and buffer arithmetic below");

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

// QN = groups of 8 tokens in use (1 .. 4): the token loop has no run-time bounds.
//
// Pipeline of one thread.  Weights: step j of the CTA's k range is fetched with two 16-byte cp.async into the
// thread's own place in slot j % kDepth of a shared-memory ring (it will read them back itself, so no barrier is
// involved) and committed as group j; before step i is multiplied, step i + kDepth - 1 is issued and
// cp.async.wait_group leaves at most kDepth - 1 groups pending, i.e. group i is complete.  Asynchronous copies are
// tracked by group, not by register scoreboards, so all seven steps ahead really are in flight (a ring of registers
// filled by plain loads is not: a warp has a handful of scoreboards, and waiting for the oldest load waits for
// younger ones on the same scoreboard too).  Activations: whenever the issue front enters a new chunk of kXSteps
// steps, all threads together fetch that chunk (every token's 512 bytes) into the activation buffer the chunk
// before last used, inside the same group; when the multiply front enters the chunk, every thread has waited for
// its own copies and one block barrier makes the chunk visible to all warps.
//
// FR = 16-row fragments per warp (1: eight warps per CTA, 2: four).  With two fragments a warp converts an
// activation vector once for both, and the per-step bookkeeping is shared: worth it when there are many token groups.
template <int QN, int FR>
__global__ void __launch_bounds__(kThreads / FR, 2) fp8_linear_skinny_kernel(const __grid_constant__ Fp8LinearParams p) {
    constexpr int T = kThreads / FR;                      // threads per CTA; FR * T 16-byte vectors per half fragment row set
    extern __shared__ __align__(128) unsigned char smem[];
    unsigned char *wring = smem;                          // [kDepth][2 * FR][T] x 16 bytes
    unsigned char *xbuf = smem + kDepth * kWSlot;         // [2][kTokens][kXRow]
    grid_dependency_sync();
    const int ks = cluster_size(), part = cluster_cta_rank();
    if (ks != p.ks) {
        if (threadIdx.x == 0) *p.status = 1;
        return;
    }
    const int tile = blockIdx.x / ks;
    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31, g = lane >> 2, t = lane & 3;
    const int n0 = tile * kTileN + warp * FR * 16;      // the warp's first fragment; the next one 16 channels on
    // this CTA's share of the k steps: contiguous, the first `extra` parts take one step more
    const int steps = p.k / kStepBytes;
    const int base = steps / ks, extra = steps % ks;
    const int s_begin = part * base + (part < extra ? part : extra);
    const int nsteps = base + (part < extra ? 1 : 0);

    float acc[FR][QN][4];
#pragma unroll
    for (int f = 0; f < FR; ++f)
#pragma unroll
        for (int q = 0; q < QN; ++q)
#pragma unroll
            for (int e = 0; e < 4; ++e) acc[f][q][e] = 0.f;

    // Row-major weights: a k step of the warp's fragment is 64 bytes of 16 rows that lie k bytes apart.  Blocked
    // weights: the same 16 x 64 bytes are one contiguous KiB (row r of the fragment at r * 64) and consecutive k steps
    // follow each other, so a warp streams its fragment's rows as one sequential run of memory.
    const size_t step_stride = p.packed ? 16 * kStepBytes : kStepBytes;
    const uint8_t *w0 = (p.packed ? p.w + static_cast<size_t>(n0 / 16) * p.k * 16 + g * kStepBytes + 16 * t
                                  : p.w + static_cast<size_t>(n0 + g) * p.k + 16 * t) + static_cast<size_t>(s_begin) * step_stride;
    const size_t half = p.packed ? static_cast<size_t>(8) * kStepBytes : static_cast<size_t>(8) * p.k;
    const size_t frag = static_cast<size_t>(16) * p.k;      // from one fragment to the next: 16 rows, in either layout
    const uint8_t *xk = p.x + static_cast<size_t>(s_begin) * kStepBytes;

    auto issue = [&](int j) {      // group j: the weights of step j and, at a chunk start, the activations of the chunk
        if (j < nsteps) {
            unsigned char *slot = wring + (j & (kDepth - 1)) * kWSlot + tid * 16;
#pragma unroll
            for (int f = 0; f < FR; ++f) {
                cp_async16(slot + (2 * f) * T * 16, w0 + f * frag, true);
                cp_async16(slot + (2 * f + 1) * T * 16, w0 + f * frag + half, true);
            }
            w0 += step_stride;
            if ((j & (kXSteps - 1)) == 0) {
                unsigned char *dst = xbuf + ((j / kXSteps) & 1) * kXBuf;
                const int left = nsteps - j < kXSteps ? nsteps - j : kXSteps;     // steps of this chunk that exist
#pragma unroll
                for (int r = 0; r < QN * FR; ++r) {
                    const int idx = tid + r * T;
                    const int tok = idx >> 5, c = idx & 31;      // 32 vectors of 16 bytes per token and chunk
                    const bool valid = tok < p.m && (c >> 2) < left;
                    cp_async16(dst + tok * kXRow + c * 16, xk + static_cast<size_t>(valid ? tok : 0) * p.k + static_cast<size_t>(j) * kStepBytes + (valid ? c * 16 : 0),
                               valid);
                }
            }
        }
        asm volatile("cp.async.commit_group;" ::: "memory");      // an empty group past the end keeps the count uniform
    };

#pragma unroll
    for (int j = 0; j < kDepth - 1; ++j) issue(j);
    for (int i = 0; i < nsteps; ++i) {
        issue(i + kDepth - 1);
        asm volatile("cp.async.wait_group %0;" ::"n"(kDepth - 1) : "memory");      // group i has landed
        if ((i & (kXSteps - 1)) == 0) __syncthreads();      // ... for every thread: the chunk's activations are visible
        const unsigned char *slot = wring + (i & (kDepth - 1)) * kWSlot + tid * 16;
        // the weights are converted once and used for every token group, an activation vector once for every fragment
        uint32_t wa[FR][8], wb[FR][8];
#pragma unroll
        for (int f = 0; f < FR; ++f) {
            e4m3x16_to_f16(*reinterpret_cast<const uint4 *>(slot + (2 * f) * T * 16), wa[f]);
            e4m3x16_to_f16(*reinterpret_cast<const uint4 *>(slot + (2 * f + 1) * T * 16), wb[f]);
        }
        const unsigned char *xs = xbuf + ((i / kXSteps) & 1) * kXBuf + g * kXRow + (i & (kXSteps - 1)) * kStepBytes + 16 * t;
#pragma unroll
        for (int q = 0; q < QN; ++q) {
            uint32_t xh[8];
            e4m3x16_to_f16(*reinterpret_cast<const uint4 *>(xs + q * 8 * kXRow), xh);
#pragma unroll
            for (int v = 0; v < 4; ++v)
#pragma unroll
                for (int f = 0; f < FR; ++f)
                    mma_f16(acc[f][q], wa[f][2 * v], wb[f][2 * v], wa[f][2 * v + 1], wb[f][2 * v + 1], xh[2 * v], xh[2 * v + 1]);
        }
    }
    asm volatile("cp.async.wait_group 0;" ::: "memory");
    __syncthreads();      // every warp is done with the ring: it becomes the partial tile

    // this CTA's partial tile: token-major, fp32 (channels of a token are contiguous, as in the output)
    float *partial = reinterpret_cast<float *>(smem);
#pragma unroll
    for (int f = 0; f < FR; ++f)
#pragma unroll
        for (int q = 0; q < QN; ++q) {
            const int ch = (warp * FR + f) * 16 + g, tok = q * 8 + 2 * t;
            partial[tok * kPartPitch + ch] = acc[f][q][0];
            partial[(tok + 1) * kPartPitch + ch] = acc[f][q][1];
            partial[tok * kPartPitch + ch + 8] = acc[f][q][2];
            partial[(tok + 1) * kPartPitch + ch + 8] = acc[f][q][3];
        }
    cluster_barrier();
    // CTA `part` finishes channels [part * per, part * per + per) of the tile: sum over the cluster in CTA order
    const int per = kTileN / ks;
    for (int e = tid; e < per * QN * 8; e += T) {
        const int ch = part * per + e % per, tok = e / per;
        float sum = 0.f;
        for (int c = 0; c < ks; ++c) sum += ld_cluster_f32(partial + tok * kPartPitch + ch, c);
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

int gpuk::fp8_frags_per_warp_tuning = 0;

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
    if (device < 0 || device >= 64) return set_last_error(GPUK_ERR_UNSUPPORTED, "fp8_linear: device index %d", device);
    // one fragment per warp (eight warps), or two (four warps) for more than 16 tokens on 4096 channels or more: measured
    // at 32 tokens, one / two fragments: n = 1280 9.1 / 10.3 us, n = 4096 14.0 / 13.1 us, n = 7168 21.8 / 21.2 us (k = 8192)
    const void *fns[8] = {reinterpret_cast<const void *>(&fp8_linear_skinny_kernel<1, 1>), reinterpret_cast<const void *>(&fp8_linear_skinny_kernel<2, 1>),
                          reinterpret_cast<const void *>(&fp8_linear_skinny_kernel<3, 1>), reinterpret_cast<const void *>(&fp8_linear_skinny_kernel<4, 1>),
                          reinterpret_cast<const void *>(&fp8_linear_skinny_kernel<1, 2>), reinterpret_cast<const void *>(&fp8_linear_skinny_kernel<2, 2>),
                          reinterpret_cast<const void *>(&fp8_linear_skinny_kernel<3, 2>), reinterpret_cast<const void *>(&fp8_linear_skinny_kernel<4, 2>)};
    {
        // first call on a device (guarded for concurrent callers): the status word, and the opt-in to more than
        // 48 KiB of dynamic shared memory for every instantiation, so that no later call has set-up left to do
        static std::mutex init_mutex;
        std::lock_guard<std::mutex> lock(init_mutex);
        if (!g_status_by_device[device]) {
            for (const void *fn : fns) {
                cudaError_t ea = cudaFuncSetAttribute(fn, cudaFuncAttributeMaxDynamicSharedMemorySize, kSmemBytes);
                if (ea != cudaSuccess)
                    return set_last_error(GPUK_ERR_CUDA, "fp8_linear: cannot opt in to %d bytes of shared memory: %s", kSmemBytes, cudaGetErrorString(ea));
            }
            int *s = nullptr;
            if (cudaMalloc(&s, sizeof(int)) != cudaSuccess) return set_last_error(GPUK_ERR_CUDA, "fp8_linear: cannot allocate the status word");
            clear_status_kernel<<<1, 1, 0, static_cast<cudaStream_t>(stream)>>>(s);
            g_status_by_device[device] = s;
        }
    }
    Fp8LinearParams p = {static_cast<const uint8_t *>(x_fp8), x_scale, static_cast<const uint8_t *>(w_fp8), w_scale,
                         static_cast<__nv_bfloat16 *>(out_bf16), m, n, k, ks, w_layout, g_status_by_device[device]};
    const int qn = (m + 7) / 8;
    const int fr = (fp8_frags_per_warp_tuning == 1 || fp8_frags_per_warp_tuning == 2) ? fp8_frags_per_warp_tuning : ((qn >= 3 && n >= 4096) ? 2 : 1);
    void *args[] = {&p};
    cudaError_t e = launch_kernel(fns[(fr - 1) * 4 + qn - 1], (n / kTileN) * ks, kThreads / fr, ks, false, args, static_cast<cudaStream_t>(stream), kSmemBytes);
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

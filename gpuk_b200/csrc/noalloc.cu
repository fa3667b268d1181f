// gpuk_selfcheck_allreduce_rms: the N-rank fused exchange, emulated on the current GPU, for
// callers that must not allocate device memory.
//
// Who needs this.  A serving process usually hands (nearly) all device memory to its own arena
// at start-up, so a later cudaMalloc from a library can fail or fragment the arena; a health
// probe that re-checks the exchange logic while the server is live, or a harness that runs
// inside such a process, therefore cannot create the workspaces that
// gpuk_emulated_allreduce_rms needs (each gpuk_ws_create allocates staging memory).  This
// entry point does the same job with no allocation at all: its staging memory is a fixed
// array compiled into the library.
//
// What it costs.  The array (kScratchBytes, about 8.5 MiB) is part of the loaded module: every
// GPU on which this library's kernels are loaded holds it until the process exits.  That fixes
// the largest message at kStaticMaxMessageBytes (32 KiB per emulated rank); larger requests
// are refused with GPUK_ERR_TOO_LARGE.
//
// Rules for callers.
//   * The first call on a device sets the array up (address lookup, fill with the rest
//     pattern, time budgets).  That first call launches a fill kernel and synchronises, so make
//     it before any stream capture.
//   * All calls on a device share the one array and it keeps what the last call left in it:
//     the exchange protocol leaves the staging at rest and keeps its call counter there, the
//     status words are cleared at the start of every call.  Two calls that overlap on the GPU
//     (different streams, or different threads) race on it: issue them one after another.
//   * Every call first waits for the previous self-check on the device and looks at its status
//     words; if that one gave up waiting (its outputs are then wrong), the array is put back
//     to its initial state before the new exchange starts.
//
// It calls no cudaMalloc / cudaFree and no allocating library routine.
#include <cuda_runtime.h>

#include <cstdio>
#include <cstring>
#include <mutex>

#include "../../include/gpuk_b200.h"
#include "kernels.cuh"
#include "launch.cuh"   // gpuk::set_last_error

using namespace gpuk;

namespace {

constexpr int64_t kStaticMaxMessageBytes = 32 << 10;              // per emulated rank
constexpr int64_t kStateBytes = 4096;                             // kMaxRanks LocalState records, 256 B apart
constexpr int64_t kSlotBytes = kStaticMaxMessageBytes;            // scatter slot and one-shot slot
constexpr int64_t kTsStride = (kMaxRanks + 1) * kSlotBytes;       // N scatter slots + gather area
constexpr int64_t kOsOff = 2 * kTsStride;
constexpr int64_t kRankBytes = kOsOff + 2 * kMaxRanks * kSlotBytes;
constexpr int64_t kScratchBytes = kStateBytes + kMaxRanks * kRankBytes;
constexpr int kMaxDevices = 64;

// The scratch memory.  In host code this name is only a handle for the runtime, never an
// address a kernel may be given: the device address comes from cudaGetSymbolAddress below.
static __device__ __align__(256) unsigned char g_static_scratch[kScratchBytes];

struct EmulatedParams {
    ArParams r[kMaxRanks];
};

template <typename T, int NR, int VPT, bool TWO_SHOT>
__global__ void __launch_bounds__(ar_max_threads<VPT, TWO_SHOT>(), 1)
    ar_selfcheck_kernel(const __grid_constant__ EmulatedParams ep, int nb) {
    __shared__ EpilogueSmem sm;
    const int rank = blockIdx.x / nb;
    ar_body<T, NR, VPT, TWO_SHOT, true>(ep.r[rank], blockIdx.x % nb, nb, sm);
}

__global__ void scratch_init_kernel(unsigned char *base, unsigned long long timeout_ns) {
    const size_t n = static_cast<size_t>(kScratchBytes - kStateBytes) / 16;
    uint4 *stage = reinterpret_cast<uint4 *>(base + kStateBytes);
    const uint4 e = make_uint4(kEmptyWord, kEmptyWord, kEmptyWord, kEmptyWord);
    for (size_t i = blockIdx.x * static_cast<size_t>(blockDim.x) + threadIdx.x; i < n; i += static_cast<size_t>(gridDim.x) * blockDim.x)
        stage[i] = e;
    if (blockIdx.x == 0 && threadIdx.x < kMaxRanks) {
        LocalState *st = reinterpret_cast<LocalState *>(base + threadIdx.x * 256);
        st->seq = 0;
        st->reserved2 = 0;
        st->abort = 0;
        st->timeout_ns = timeout_ns;
        for (int i = 0; i < kStatusWords; ++i) st->status[i] = 0;
    }
}

__global__ void scratch_clear_status_kernel(unsigned char *base, int world) {
    if (threadIdx.x < world) {
        LocalState *st = reinterpret_cast<LocalState *>(base + threadIdx.x * 256);
        st->abort = 0;
        for (int i = 0; i < kStatusWords; ++i) st->status[i] = 0;
    }
}

template <typename T, int NR>
const void *kernel_for(int vpt, bool two_shot) {
    if (vpt == 1) return two_shot ? reinterpret_cast<const void *>(&ar_selfcheck_kernel<T, NR, 1, true>)
                                  : reinterpret_cast<const void *>(&ar_selfcheck_kernel<T, NR, 1, false>);
    if (vpt == 2) return two_shot ? reinterpret_cast<const void *>(&ar_selfcheck_kernel<T, NR, 2, true>)
                                  : reinterpret_cast<const void *>(&ar_selfcheck_kernel<T, NR, 2, false>);
    if (vpt == 4) return two_shot ? reinterpret_cast<const void *>(&ar_selfcheck_kernel<T, NR, 4, true>)
                                  : reinterpret_cast<const void *>(&ar_selfcheck_kernel<T, NR, 4, false>);
    return nullptr;
}

template <typename T>
const void *kernel_for_world(int world, int vpt, bool two_shot) {
    switch (world) {
    case 2: return kernel_for<T, 2>(vpt, two_shot);
    case 4: return kernel_for<T, 4>(vpt, two_shot);
    case 8: return kernel_for<T, 8>(vpt, two_shot);
    default: return nullptr;
    }
}

// Per-device set-up state (host side).
struct DeviceScratch {
    unsigned char *base = nullptr;   // device address of g_static_scratch on that device
    bool dirty = false;              // needs (re-)initialisation before the next exchange
};
DeviceScratch g_dev[kMaxDevices];
std::mutex g_mu;

}  // namespace

extern "C" int gpuk_selfcheck_allreduce_rms(int world_size, void *const *allreduce_in, const void *residual_in,
                                            const void *rms_gamma, void *const *residual_out, void *const *norm_out,
                                            float *const *scale_out, int64_t numel, int hidden, int dtype, float eps,
                                            int quant_type, int force_mode, void *stream) {
    if (!allreduce_in || !residual_in || !rms_gamma || !residual_out || !norm_out)
        return set_last_error(GPUK_ERR_INVALID_ARGUMENT, "selfcheck: null argument");
    if (world_size != 2 && world_size != 4 && world_size != 8)
        return set_last_error(GPUK_ERR_INVALID_ARGUMENT, "world size is not supported");
    if (hidden <= 0) return set_last_error(GPUK_ERR_INVALID_ARGUMENT, "selfcheck: hidden must be positive");
    if (numel == 0) return GPUK_OK;

    Quant q;
    switch (quant_type) {
    case GPUK_QUANT_NONE: q = {kQuantNone, 0, 0.f}; break;
    case GPUK_QUANT_FP8_E4M3FN_240: q = {kQuantDynamic, 0, 240.f}; break;
    case GPUK_QUANT_FP8_E4M3FNUZ_120: q = {kQuantDynamic, 1, 120.f}; break;
    case GPUK_QUANT_FP8_E4M3FN_448: q = {kQuantDynamic, 0, 448.f}; break;
    case GPUK_QUANT_FP8_E4M3FN_448_STATIC: q = {kQuantStatic, 0, 448.f}; break;
    default: return set_last_error(GPUK_ERR_INVALID_ARGUMENT, "unknown quant_type %d", quant_type);
    }
    if (q.mode != kQuantNone && !scale_out) return set_last_error(GPUK_ERR_INVALID_ARGUMENT, "selfcheck: scale_out is null");

    // shape -> tile, through the library's own planner (pure host arithmetic)
    int device = 0, sms = 0;
    if (cudaGetDevice(&device) != cudaSuccess || device < 0 || device >= kMaxDevices)
        return set_last_error(GPUK_ERR_CUDA, "selfcheck: no current CUDA device");
    cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, device);
    gpuk_plan plan;
    const int64_t crossover = force_mode == 1 ? kStaticMaxMessageBytes : (force_mode == 2 ? 1 : 0);
    int rc = gpuk_plan_allreduce_rms(world_size, numel, hidden, dtype, sms, 0, crossover, &plan);
    if (rc) return rc;
    if (plan.message_bytes > kStaticMaxMessageBytes)
        return set_last_error(GPUK_ERR_TOO_LARGE,
                              "selfcheck: message of %lld bytes per rank exceeds the built-in scratch (limit %lld bytes); "
                              "use gpuk_emulated_allreduce_rms with workspaces for larger cases",
                              (long long)plan.message_bytes, (long long)kStaticMaxMessageBytes);
    if (plan.vpt > 4)
        return set_last_error(GPUK_ERR_UNSUPPORTED, "selfcheck: rows of %d vectors are not built for the no-allocation variant", plan.row_vecs);
    const bool two_shot = plan.one_shot == 0;

    const void *fn = nullptr;
    switch (dtype) {
    case GPUK_DTYPE_BF16: fn = kernel_for_world<__nv_bfloat16>(world_size, plan.vpt, two_shot); break;
    case GPUK_DTYPE_F16: fn = kernel_for_world<__half>(world_size, plan.vpt, two_shot); break;
    case GPUK_DTYPE_F32: fn = kernel_for_world<float>(world_size, plan.vpt, two_shot); break;
    default: break;
    }
    if (!fn) return set_last_error(GPUK_ERR_UNSUPPORTED, "selfcheck: no kernel for this dtype / tile");

    cudaStream_t s = static_cast<cudaStream_t>(stream);
    unsigned char *base = nullptr;
    {
        // once per device, with that device current: the device address of the scratch array
        std::lock_guard<std::mutex> lock(g_mu);
        DeviceScratch &d = g_dev[device];
        if (!d.base) {
            void *p = nullptr;
            cudaError_t e = cudaGetSymbolAddress(&p, g_static_scratch);
            if (e != cudaSuccess || !p)
                return set_last_error(GPUK_ERR_CUDA, "selfcheck: cudaGetSymbolAddress failed: %s", cudaGetErrorString(e));
            d.base = static_cast<unsigned char *>(p);
            d.dirty = true;
        }
        if (!d.dirty) {
            // did the previous self-check on this device give up?  (waits for it to finish)
            alignas(16) unsigned char states[kStateBytes];
            cudaError_t e = cudaMemcpy(states, d.base, kStateBytes, cudaMemcpyDeviceToHost);
            if (e != cudaSuccess) return set_last_error(GPUK_ERR_CUDA, "selfcheck: reading the scratch state failed: %s", cudaGetErrorString(e));
            for (int r = 0; r < kMaxRanks; ++r)
                if (reinterpret_cast<const LocalState *>(states + r * 256)->status[0] != 0) d.dirty = true;
        }
        if (d.dirty) {
            scratch_init_kernel<<<296, 256, 0, s>>>(d.base, 2000000000ull);
            cudaError_t e = cudaGetLastError();
            if (e == cudaSuccess) e = cudaStreamSynchronize(s);
            if (e != cudaSuccess) return set_last_error(GPUK_ERR_CUDA, "selfcheck: scratch set-up failed: %s", cudaGetErrorString(e));
            d.dirty = false;
        }
        base = d.base;
    }

    // co-residency: all emulated ranks' CTAs wait for each other inside one launch
    int64_t resident = 0;
    cudaError_t e = resident_ctas(fn, plan.threads, plan.cluster, sms, &resident);
    if (e != cudaSuccess || resident <= 0) return set_last_error(GPUK_ERR_CUDA, "selfcheck: occupancy query failed");
    int64_t clusters = resident / world_size / plan.cluster;
    if (clusters > plan.rows) clusters = plan.rows;
    if (clusters > plan.grid / plan.cluster) clusters = plan.grid / plan.cluster;
    if (clusters < 1) return set_last_error(GPUK_ERR_UNSUPPORTED, "selfcheck: the GPU cannot hold one cluster per emulated rank");
    const int64_t nb = clusters * plan.cluster;

    const int es = dtype == GPUK_DTYPE_F32 ? 4 : 2;
    EmulatedParams ep;
    memset(&ep, 0, sizeof(ep));
    for (int r = 0; r < world_size; ++r) {
        ArParams &p = ep.r[r];
        if (!allreduce_in[r] || !residual_out[r] || !norm_out[r])
            return set_last_error(GPUK_ERR_INVALID_ARGUMENT, "selfcheck: null tensor pointer for rank %d", r);
        const uintptr_t bits = reinterpret_cast<uintptr_t>(allreduce_in[r]) | reinterpret_cast<uintptr_t>(residual_out[r]) |
                               reinterpret_cast<uintptr_t>(norm_out[r]) | reinterpret_cast<uintptr_t>(residual_in) |
                               reinterpret_cast<uintptr_t>(rms_gamma);
        if (bits & 15u) return set_last_error(GPUK_ERR_INVALID_ARGUMENT, "tensor pointers must be 16-byte aligned");
        p.in = allreduce_in[r];
        p.out = allreduce_in[r];
        p.total_vecs = numel * es / 16;
        p.rows = plan.rows;
        p.row_vecs = plan.row_vecs;
        p.rows_per_chunk = 1;
        p.seg_vecs = (plan.row_vecs + plan.cluster - 1) / plan.cluster;
        p.lead_push = plan.lead_push > 0 ? plan.lead_push : 1;
        p.lead_reduce = plan.lead_reduce > 0 ? plan.lead_reduce : 1;
        p.ep.residual = residual_in;
        p.ep.gamma = rms_gamma;
        p.ep.residual_out = residual_out[r];
        p.ep.norm_out = norm_out[r];
        p.ep.scale_out = scale_out ? scale_out[r] : nullptr;
        p.ep.hidden = hidden;
        p.ep.row_vecs = plan.row_vecs;
        p.ep.eps = eps;
        p.ep.q = q;
        p.rank = r;
        p.vpr = (plan.row_vecs + world_size - 1) / world_size;
        for (int j = 0; j < world_size; ++j) p.peer_data[j] = reinterpret_cast<char *>(base + kStateBytes + j * kRankBytes);
        p.st = reinterpret_cast<LocalState *>(base + r * 256);
        p.rs_slot_bytes = kSlotBytes;
        p.ag_off = kMaxRanks * kSlotBytes;
        p.ts_stride = kTsStride;
        p.os_off = kOsOff;
        p.os_slot_bytes = kSlotBytes;
    }

    scratch_clear_status_kernel<<<1, 32, 0, s>>>(base, world_size);
    int nb_arg = static_cast<int>(nb);
    void *args[] = {&ep, &nb_arg};
    e = launch_kernel(fn, static_cast<int>(nb * world_size), plan.threads, plan.cluster, true, args, s);
    if (e != cudaSuccess) return set_last_error(GPUK_ERR_CUDA, "selfcheck: launch failed: %s", cudaGetErrorString(e));
    return GPUK_OK;
}

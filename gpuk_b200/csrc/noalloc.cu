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
//     pattern, time budgets).  That first call launches a fill kernel and synchronises the
//     stream, so make it before any stream capture (during a capture it is refused).
//   * All calls on a device share the one array and it keeps what the last call left in it:
//     the exchange protocol leaves the staging at rest, one call counter for all emulated ranks
//     lives there, and the status words are cleared at the start of every call.  Two calls that
//     overlap on the GPU (different streams, or different threads) race on it: issue them one
//     after another on one stream.
//   * Later calls are plain stream-ordered launches.  Each begins with a small kernel that looks
//     at the status words the previous call left; if that call gave up waiting (its outputs are
//     then wrong), the staging is put back to rest on the device before the new exchange starts.
//   * gpuk_selfcheck_status tells the caller whether its own call completed: it waits for the
//     stream and returns the status words of the last call (also without allocating).
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
constexpr int64_t kStateBytes = 4096;                             // kMaxRanks LocalState records, 256 B apart, then the call counter
constexpr int64_t kCallCountOff = kMaxRanks * 256;                // one 64-bit count of exchanges for ALL emulated ranks
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

__device__ __forceinline__ void fill_staging_at_rest(unsigned char *base) {
    const size_t n = static_cast<size_t>(kScratchBytes - kStateBytes) / 16;
    uint4 *stage = reinterpret_cast<uint4 *>(base + kStateBytes);
    const uint4 e = make_uint4(kEmptyWord, kEmptyWord, kEmptyWord, kEmptyWord);
    for (size_t i = blockIdx.x * static_cast<size_t>(blockDim.x) + threadIdx.x; i < n; i += static_cast<size_t>(gridDim.x) * blockDim.x)
        stage[i] = e;
}

__global__ void scratch_init_kernel(unsigned char *base, unsigned long long timeout_ns) {
    fill_staging_at_rest(base);
    if (blockIdx.x == 0 && threadIdx.x < kMaxRanks) {
        LocalState *st = reinterpret_cast<LocalState *>(base + threadIdx.x * 256);
        st->seq = 0;
        st->reserved2 = 0;
        st->abort = 0;
        st->timeout_ns = timeout_ns;
        for (int i = 0; i < kStatusWords; ++i) st->status[i] = 0;
    }
    if (blockIdx.x == 0 && threadIdx.x == 0) *reinterpret_cast<unsigned long long *>(base + kCallCountOff) = 0ull;
}

// First kernel of every call: if the previous call on this device gave up (any status word set),
// the staging may hold unconsumed vectors and goes back to rest.  Status words are only read here.
__global__ void scratch_repair_kernel(unsigned char *base) {
    bool bad = false;
    for (int r = 0; r < kMaxRanks; ++r) bad |= reinterpret_cast<const LocalState *>(base + r * 256)->status[0] != 0;
    if (bad) fill_staging_at_rest(base);
}

// Second kernel of every call: clears the status words and gives EVERY emulated rank the same call
// number.  The low bit of that number selects the staging buffer, so ranks that sat out earlier
// calls (a smaller world size) must not keep a stale one.
__global__ void scratch_begin_call_kernel(unsigned char *base) {
    unsigned long long *count = reinterpret_cast<unsigned long long *>(base + kCallCountOff);
    const unsigned long long c = *count;
    __syncthreads();
    if (threadIdx.x < kMaxRanks) {
        LocalState *st = reinterpret_cast<LocalState *>(base + threadIdx.x * 256);
        st->seq = c << 16;
        st->abort = 0;
        for (int i = 0; i < kStatusWords; ++i) st->status[i] = 0;
    }
    if (threadIdx.x == 0) *count = c + 1;
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
    bool ready = false;              // set-up done (array at rest, time budgets written)
};
DeviceScratch g_dev[kMaxDevices];
std::mutex g_mu;

// Device address of the scratch array on `device` (which must be current); the first call per
// device looks it up and puts the array into its initial state (synchronises `s`).
int scratch_base(int device, cudaStream_t s, unsigned char **out) {
    std::lock_guard<std::mutex> lock(g_mu);
    DeviceScratch &d = g_dev[device];
    if (!d.base) {
        // in host code the array's name is a stand-in, not an address: ask the runtime for it
        void *p = nullptr;
        cudaError_t e = cudaGetSymbolAddress(&p, g_static_scratch);
        if (e != cudaSuccess || !p)
            return set_last_error(GPUK_ERR_CUDA, "selfcheck: cudaGetSymbolAddress failed: %s", cudaGetErrorString(e));
        d.base = static_cast<unsigned char *>(p);
    }
    if (!d.ready) {
        cudaStreamCaptureStatus cap = cudaStreamCaptureStatusNone;
        if (cudaStreamIsCapturing(s, &cap) != cudaSuccess) cudaGetLastError();
        if (cap != cudaStreamCaptureStatusNone)
            return set_last_error(GPUK_ERR_INVALID_ARGUMENT, "selfcheck: the first call on a device sets the scratch array up and "
                                                             "synchronises; make it before the stream capture begins");
        scratch_init_kernel<<<296, 256, 0, s>>>(d.base, 2000000000ull);
        cudaError_t e = cudaGetLastError();
        if (e == cudaSuccess) e = cudaStreamSynchronize(s);
        if (e != cudaSuccess) return set_last_error(GPUK_ERR_CUDA, "selfcheck: scratch set-up failed: %s", cudaGetErrorString(e));
        d.ready = true;
    }
    *out = d.base;
    return GPUK_OK;
}

}  // namespace

extern "C" int gpuk_selfcheck_status(uint32_t out[8], void *stream) {
    if (!out) return set_last_error(GPUK_ERR_INVALID_ARGUMENT, "selfcheck: null output");
    int device = 0;
    if (cudaGetDevice(&device) != cudaSuccess || device < 0 || device >= kMaxDevices)
        return set_last_error(GPUK_ERR_CUDA, "selfcheck: no current CUDA device");
    cudaStream_t s = static_cast<cudaStream_t>(stream);
    memset(out, 0, sizeof(uint32_t) * kStatusWords);
    unsigned char *base = nullptr;
    {
        std::lock_guard<std::mutex> lock(g_mu);
        if (!g_dev[device].ready) return GPUK_OK;   // no self-check has run on this device
        base = g_dev[device].base;
    }
    alignas(16) unsigned char states[kMaxRanks * 256];
    cudaError_t e = cudaMemcpyAsync(states, base, sizeof(states), cudaMemcpyDeviceToHost, s);
    if (e == cudaSuccess) e = cudaStreamSynchronize(s);
    if (e != cudaSuccess) return set_last_error(GPUK_ERR_CUDA, "selfcheck: reading the status words failed: %s", cudaGetErrorString(e));
    for (int r = 0; r < kMaxRanks; ++r) {
        const LocalState *st = reinterpret_cast<const LocalState *>(states + r * 256);
        if (st->status[0] != 0) {
            memcpy(out, st->status, sizeof(uint32_t) * kStatusWords);
            if (out[0] == kStatusClusterMismatch)
                return set_last_error(GPUK_ERR_BAD_LAUNCH, "selfcheck: emulated rank %u CTA %u ran in a thread-block cluster of %u CTAs, "
                                      "not the planned size; nothing was written", out[1], out[2], out[6]);
            return set_last_error(GPUK_ERR_PEER_TIMEOUT, "selfcheck: emulated rank %u CTA %u thread %u gave up waiting for data from rank %u "
                                  "in stage %u (word seen 0x%08x)", out[1], out[2], out[5], out[4], out[3], out[6]);
        }
    }
    return GPUK_OK;
}

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
    if (!quant_from_type(quant_type, &q)) return set_last_error(GPUK_ERR_INVALID_ARGUMENT, "unknown quant_type %d", quant_type);
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
    rc = scratch_base(device, s, &base);
    if (rc) return rc;

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
        p.cluster = plan.cluster;
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
        p.ep.hidden_f = static_cast<float>(hidden);
        p.ep.inv_hidden = static_cast<float>(1.0 / static_cast<double>(hidden));
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

    scratch_repair_kernel<<<296, 256, 0, s>>>(base);
    scratch_begin_call_kernel<<<1, 32, 0, s>>>(base);
    e = cudaGetLastError();
    if (e != cudaSuccess) return set_last_error(GPUK_ERR_CUDA, "selfcheck: launch failed: %s", cudaGetErrorString(e));
    int nb_arg = static_cast<int>(nb);
    void *args[] = {&ep, &nb_arg};
    e = launch_kernel(fn, static_cast<int>(nb * world_size), plan.threads, plan.cluster, true, args, s);
    if (e != cudaSuccess) return set_last_error(GPUK_ERR_CUDA, "selfcheck: launch failed: %s", cudaGetErrorString(e));
    return GPUK_OK;
}

// Host side of the C ABI declared in include/gpuk_b200.h: the per-rank workspace (staging
// memory, flag array, device-resident state), CUDA-IPC export/import, the launch policy and
// the entry points.  Replaces src/ops/all_reduce_fusion.cpp:4-396 of the reference.
//
// Workspace memory of one rank (one cudaMalloc, exported as one IPC handle), everything
// double-buffered by call parity and at rest filled with kEmptyWord (common.cuh):
//
//   two-shot buffer b at b*ts_stride:
//     [0, N*rs_slot)            scatter slots: slot s holds, for every row, the column slice this
//                               rank owns as pushed by rank s
//     [ag_off, ag_off + cap)    gather area: the reduced tensor, same layout as the input
//   one-shot buffer b at os_off + b*N*os_slot: slot s holds rank s's whole message
//   the last 256 bytes are never written by any exchange (used by the wait self-test)
//
// A second, small allocation is exported through the "barrier handle" calls of the operator
// API; the exchange needs no flags, its words are reserved.  The device-resident LocalState
// (call counter, ticket, status) is never exported.
#include <cuda.h>
#include <cuda_runtime.h>

#include <algorithm>
#include <cstdarg>
#include <cstdio>
#include <cstdlib>
#include <cstring>
#include <map>
#include <new>
#include <string>
#include <type_traits>
#include <vector>

#include "../../include/gpuk_b200.h"
#include "launch.cuh"

using namespace gpuk;

namespace {

thread_local std::string g_last_error;

int fail(int code, const char *fmt, ...) {
    char buf[512];
    va_list ap;
    va_start(ap, fmt);
    vsnprintf(buf, sizeof(buf), fmt, ap);
    va_end(ap);
    g_last_error = buf;
    return code;
}

}  // namespace

int gpuk::set_last_error(int code, const char *fmt, ...) {
    char buf[512];
    va_list ap;
    va_start(ap, fmt);
    vsnprintf(buf, sizeof(buf), fmt, ap);
    va_end(ap);
    g_last_error = buf;
    return code;
}

cudaError_t gpuk::launch_kernel(const void *fn, int grid, int threads, int cluster, bool all_resident, void **args,
                                cudaStream_t stream, size_t dynamic_smem) {
    // A grid that must be resident as a whole is launched cooperatively, which the driver refuses
    // when it does not fit.  The cooperative attribute is never combined with a cluster dimension
    // (the combination is not honoured everywhere: a launch can be accepted and run without its
    // cluster): a clustered all-resident launch carries the cluster attribute alone, its callers
    // size the grid in whole clusters with resident_ctas(), and every wait in the kernels is bounded.
    if (cluster <= 1 && all_resident) return cudaLaunchCooperativeKernel(fn, dim3(grid), dim3(threads), args, dynamic_smem, stream);
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = dim3(grid);
    cfg.blockDim = dim3(threads);
    cfg.dynamicSmemBytes = dynamic_smem;
    cfg.stream = stream;
    cudaLaunchAttribute attrs[2];
    int n = 0;
    if (cluster > 1) {
        attrs[n].id = cudaLaunchAttributeClusterDimension;
        attrs[n].val.clusterDim.x = cluster;
        attrs[n].val.clusterDim.y = 1;
        attrs[n].val.clusterDim.z = 1;
        ++n;
    }
    if (!all_resident) {
        attrs[n].id = cudaLaunchAttributeProgrammaticStreamSerialization;
        attrs[n].val.programmaticStreamSerializationAllowed = 1;
        ++n;
    }
    cfg.attrs = attrs;
    cfg.numAttrs = n;
    return cudaLaunchKernelExC(&cfg, fn, args);
}

cudaError_t gpuk::resident_ctas(const void *fn, int threads, int cluster, int sm_count, int64_t *ctas) {
    if (cluster <= 1) {
        int per_sm = 0;
        cudaError_t e = cudaOccupancyMaxActiveBlocksPerMultiprocessor(&per_sm, fn, threads, 0);
        *ctas = static_cast<int64_t>(per_sm) * sm_count;
        return e;
    }
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = dim3(cluster * sm_count);
    cfg.blockDim = dim3(threads);
    cudaLaunchAttribute attr;
    attr.id = cudaLaunchAttributeClusterDimension;
    attr.val.clusterDim.x = cluster;
    attr.val.clusterDim.y = 1;
    attr.val.clusterDim.z = 1;
    cfg.attrs = &attr;
    cfg.numAttrs = 1;
    int clusters = 0;
    cudaError_t e = cudaOccupancyMaxActiveClusters(&clusters, fn, &cfg);
    *ctas = static_cast<int64_t>(clusters) * cluster;
    return e;
}

namespace {

#define GPUK_CUDA(expr)                                                                            \
    do {                                                                                           \
        cudaError_t err__ = (expr);                                                                \
        if (err__ != cudaSuccess)                                                                  \
            return fail(GPUK_ERR_CUDA, "%s failed: %s (%s:%d)", #expr, cudaGetErrorString(err__), \
                        __FILE__, __LINE__);                                                       \
    } while (0)

constexpr int kDefaultSmCount = 148;            // B200
constexpr int64_t kOneShotSlotBytes = 2 << 20;  // largest one-shot message
constexpr int64_t kRsSlack = 1 << 20;           // room for ceil(row_vecs / N) rounding in the RS slots
constexpr uint64_t kDefaultTimeoutNs = 2000000000ull;
constexpr size_t kFlagBytes = 4096;             // the allocation behind the "barrier handle"
constexpr int64_t kTailBytes = 256;             // never written by an exchange
constexpr int kPlainRowVecs = 1024;             // the plain all-reduce views its input as 16 KiB rows
// The one-GPU kernel for many rows (persistent CTAs, rows staged through shared memory).  Measured on
// B200 at hidden 8192, fraction of the HBM copy peak, one row per CTA / staged with 512 threads and two
// stages: 1024 rows 0.70 / 0.63, 2048 rows 0.84 / 0.82, 4096 rows 0.89 / 0.93, 16384 x 7168 0.97 / 0.98.
constexpr int kDefaultK1Threads = 512;          // preferred CTA size of that kernel
constexpr int kDefaultK1Stages = 2;             // its shared-memory stages (0: never use it)
constexpr int64_t kK1StagedMinRows(int sms) { return 20ll * sms; }   // ... used from this many rows

// process-wide tuning of the one-GPU kernel (gpuk_set_tuning); negative / zero: built-in choice
struct Tuning {
    int k1_stages = -1;
    int64_t k1_staged_min_rows = -1;
    int k1_ctas_per_sm = 0;
    int k1_threads = 0;       // preferred CTA size of the persistent variant
};
Tuning g_tuning;
constexpr int kWsFinishThreads = 512;           // warp-specialised two-shot kernel: threads per role (kernels.cuh: kWsMaxThreads)
constexpr int kWsScatterLeadShort = 2;          // ... rows the scatter may run ahead of the finish: few rows per CTA / many
constexpr int kWsScatterLeadLong = 8;
constexpr int kWsReduceThreads = 128;
constexpr int kWsScatterThreads = 128;
constexpr int kDefaultLeadPush = 1;             // two-shot pipeline depths (chunks), see ar_body
constexpr int kDefaultLeadReduce = 1;

int elem_size(int dtype) {
    switch (dtype) {
    case GPUK_DTYPE_BF16:
    case GPUK_DTYPE_F16: return 2;
    case GPUK_DTYPE_F32: return 4;
    default: return 0;
    }
}

bool valid_world(int w) { return w == 2 || w == 4 || w == 8; }

int64_t default_oneshot_max_bytes(int world) {
    // The reference's rule is impl.h:375-376.  Measured on B200 at hidden 8192 (CUDA-graph replay, us per
    // call, one-shot / two-shot): two ranks 10.0 / 13.5 at 2 MiB; eight ranks 12.3 / 15.5 at 256 KiB,
    // 15.5 / 16.1 at 512 KiB, 20.8 / 14.3 at 1 MiB.  Four ranks: between the two.
    switch (world) {
    case 2: return 2 << 20;
    case 4: return 1 << 20;
    default: return 512 << 10;
    }
}

}  // namespace
bool gpuk::quant_from_type(int quant_type, Quant *q) {
    switch (quant_type) {
    case GPUK_QUANT_NONE: *q = make_quant(kQuantNone, 0, 0.f); return true;
    case GPUK_QUANT_FP8_E4M3FN_240: *q = make_quant(kQuantDynamic, 0, 240.f); return true;
    case GPUK_QUANT_FP8_E4M3FNUZ_120: *q = make_quant(kQuantDynamic, 1, 120.f); return true;
    case GPUK_QUANT_FP8_E4M3FN_448: *q = make_quant(kQuantDynamic, 0, 448.f); return true;
    case GPUK_QUANT_FP8_E4M3FN_448_STATIC: *q = make_quant(kQuantStatic, 0, 448.f); return true;
    default: return false;
    }
}
namespace {

bool aligned16(const void *p) { return (reinterpret_cast<uintptr_t>(p) & 15u) == 0; }

int max_threads_for(int vpt) { return vpt == 4 ? 256 : (vpt == 8 ? 512 : 1024); }   // kernels.cuh: tile_max_threads

// Tile of a row: `vpt` 16-byte vectors per thread, `threads` per CTA.
bool pick_tile(int row_vecs, bool latency, int *vpt, int *threads) {
    const int target = latency ? 1024 : 256;
    int v = 1;
    while (v < 8 && row_vecs > v * target) v *= 2;
    while ((row_vecs + v - 1) / v > max_threads_for(v)) {
        if (v == 8) return false;
        v *= 2;
    }
    int t = (row_vecs + v - 1) / v;
    t = (t + 31) / 32 * 32;
    *vpt = v;
    *threads = t;
    return true;
}

}  // namespace

namespace {
__global__ void fill_empty_kernel(uint4 *p, size_t n) {
    const uint4 e = make_uint4(kEmptyWord, kEmptyWord, kEmptyWord, kEmptyWord);
    for (size_t i = blockIdx.x * static_cast<size_t>(blockDim.x) + threadIdx.x; i < n; i += static_cast<size_t>(gridDim.x) * blockDim.x) p[i] = e;
}
// Puts staging memory into its rest state (synchronous).
cudaError_t fill_empty(void *p, int64_t bytes) {
    fill_empty_kernel<<<1184, 256>>>(static_cast<uint4 *>(p), static_cast<size_t>(bytes / 16));
    cudaError_t e = cudaGetLastError();
    return e == cudaSuccess ? cudaDeviceSynchronize() : e;
}
}  // namespace

struct gpuk_ws {
    int device = 0, rank = 0, world = 0;
    int sm_count = kDefaultSmCount;
    int64_t cap = 0;            // largest message in bytes
    int64_t rs_slot_bytes = 0, ag_off = 0, ts_stride = 0, os_off = 0, os_slot_bytes = 0, data_bytes = 0;
    char *data = nullptr;
    uint32_t *flags = nullptr;
    LocalState *st = nullptr;
    ArParams *emul_params = nullptr;   // device scratch for the one-GPU emulation (lazily allocated)
    void *peer_data[kMaxRanks] = {};
    void *peer_flags[kMaxRanks] = {};
    bool have_data = false, have_flags = false;
    std::vector<void *> ipc_opened;
    int64_t oneshot_max_bytes = 0;
    int opt_rows_per_chunk = 0, opt_ctas_per_sm = 0;   // 0 = default
    int opt_lead_push = 0, opt_lead_reduce = 0;
    int opt_cluster = 0;                 // CTAs per row (0: the planner decides)
    int opt_ws_scatter_lead = -1;        // rows its scatter may run ahead of its finish (-1: default, 0: unbounded)
    int opt_ws_tf = 0, opt_ws_tr = 0, opt_ws_ts = 0;   // threads per role of that kernel (0: default)
    int opt_two_shot_ws = 1;             // 1: two-shot calls without clusters run the warp-specialised kernel
    int opt_two_rank_one_hop = 1;        // 1: at two ranks that kernel sends whole rows to the peer (one hop) instead of slices (two)
    bool test_withhold_cluster = false;  // test hook: launch without the planned cluster attribute
    // exchange through symmetric memory (gpuk_ws_attach_symmetric)
    char *sym[kMaxRanks] = {};
    char *sym_mc = nullptr;
    int64_t sym_cap = 0, sym_flag_off = 0;   // largest message; offset of the flags
    int64_t sym_min_bytes = 0;               // messages from this size take it (0: never automatically)
    bool sym_use_mc = true;                  // reduce inside the switch where a multicast mapping exists
    const uint32_t *ready = nullptr;         // row-block ready words of the NEXT fused call's input (gpuk_ws_set_ready_words)
    int ready_rows = 0;
    uint32_t ready_value = 0;
    int opt_ws_max_ctas = 0;                 // CTAs (= SMs) the warp-specialised kernel may take (0: all)
    bool gather_multicast = false;           // two-shot gather through the multicast address (symmetric memory holds the gather areas)
    std::map<uint32_t, int64_t> occupancy;   // CTAs resident on the whole GPU, by kernel instantiation
};

extern "C" {

const char *gpuk_last_error(void) { return g_last_error.c_str(); }

const char *gpuk_status_string(int status) {
    switch (status) {
    case GPUK_OK: return "ok";
    case GPUK_ERR_INVALID_ARGUMENT: return "invalid argument";
    case GPUK_ERR_CUDA: return "CUDA runtime error";
    case GPUK_ERR_UNSUPPORTED: return "unsupported shape or dtype";
    case GPUK_ERR_NOT_READY: return "peer memory not opened";
    case GPUK_ERR_TOO_LARGE: return "message larger than the workspace";
    case GPUK_ERR_PEER_TIMEOUT: return "timed out waiting for a peer";
    case GPUK_ERR_BAD_LAUNCH: return "kernel ran in another launch shape than planned";
    default: return "unknown status";
    }
}

// ---------------------------------------------------------------------------------------
// planning (pure host arithmetic)
// ---------------------------------------------------------------------------------------
// Per-workspace overrides of the planner's choices (gpuk_ws_set_option); 0 = the planner decides.
struct PlanOverrides {
    int cluster = 0;          // CTAs per row: 1, 2, 4 or 8
    int rows_per_chunk = 0;
    bool allow_cluster = true;   // false: every row stays in one CTA (the exchange through symmetric memory)
    bool allow_ws = true;        // false: never the warp-specialised two-shot kernel
    int ws_tf = 0, ws_tr = 0, ws_ts = 0;   // its threads per role (0: default)
};

static int plan_call(int world_size, int64_t numel, int hidden, int dtype, int sm_count, int ctas_per_sm_limit,
                     int64_t oneshot_max_bytes, const PlanOverrides &ov, gpuk_plan *out);

int gpuk_plan_allreduce_rms(int world_size, int64_t numel, int hidden, int dtype, int sm_count,
                            int ctas_per_sm_limit, int64_t oneshot_max_bytes, gpuk_plan *out) {
    return plan_call(world_size, numel, hidden, dtype, sm_count, ctas_per_sm_limit, oneshot_max_bytes, PlanOverrides(), out);
}

static int plan_call(int world_size, int64_t numel, int hidden, int dtype, int sm_count, int ctas_per_sm_limit,
                     int64_t oneshot_max_bytes, const PlanOverrides &ov, gpuk_plan *out) {
    if (!out) return fail(GPUK_ERR_INVALID_ARGUMENT, "plan: out is null");
    const int es = elem_size(dtype);
    if (!es) return fail(GPUK_ERR_UNSUPPORTED, "plan: unknown dtype %d", dtype);
    if (world_size != 1 && !valid_world(world_size))
        return fail(GPUK_ERR_INVALID_ARGUMENT, "plan: world size %d is not 1, 2, 4 or 8", world_size);
    if (numel < 0) return fail(GPUK_ERR_INVALID_ARGUMENT, "plan: negative numel");
    if (sm_count <= 0) sm_count = kDefaultSmCount;
    const int kv = 16 / es;
    const bool fused = hidden > 0;
    int row_vecs;
    int64_t rows;
    if (fused) {
        if (hidden % kv) return fail(GPUK_ERR_UNSUPPORTED, "hidden %d is not a multiple of %d elements (16 bytes)", hidden, kv);
        if (numel % hidden) return fail(GPUK_ERR_INVALID_ARGUMENT, "numel %lld is not a multiple of hidden %d", (long long)numel, hidden);
        row_vecs = hidden / kv;
        rows = numel / hidden;
    } else {
        if (numel % kv) return fail(GPUK_ERR_UNSUPPORTED, "numel %lld is not a multiple of %d elements (16 bytes)", (long long)numel, kv);
        const int64_t total_vecs = numel / kv;
        row_vecs = static_cast<int>(std::min<int64_t>(std::max<int64_t>(total_vecs, 1), kPlainRowVecs));
        rows = (total_vecs + row_vecs - 1) / row_vecs;
    }
    if (rows > (1ll << 30)) return fail(GPUK_ERR_UNSUPPORTED, "too many rows");
    const int64_t bytes = numel * es;
    if (oneshot_max_bytes <= 0) oneshot_max_bytes = world_size > 1 ? default_oneshot_max_bytes(world_size) : 0;
    const bool one_shot = world_size > 1 && bytes <= std::min(oneshot_max_bytes, kOneShotSlotBytes) && rows <= kMaxBlocks;
    const bool latency = rows <= sm_count;
    // Few rows: a row is split over the CTAs of a thread-block cluster so that the exchange runs on
    // many SMs, as long as a CTA keeps at least 128 vectors.
    int cluster = 1;
    if (world_size > 1 && fused && ov.allow_cluster) {
        while (cluster < 8 && (row_vecs + 2 * cluster - 1) / (2 * cluster) >= 128 && rows * 2 * cluster <= 2ll * sm_count) cluster *= 2;
        if (ov.cluster == 1 || ov.cluster == 2 || ov.cluster == 4 || ov.cluster == 8) cluster = ov.cluster;
        while (cluster > 1 && (row_vecs + cluster - 1) / cluster < 32) cluster /= 2;
    }
    const int seg_vecs = (row_vecs + cluster - 1) / cluster;
    int vpt = 4, threads = 256;
    if (fused || one_shot) {
        // the row must fit one CTA's tile whichever exchange is chosen, clusters or not
        // (the two-shot kernels are built for the bandwidth tile only)
        const bool wide = latency && (one_shot || world_size == 1);
        if (!pick_tile(row_vecs, wide, &vpt, &threads) || !pick_tile(seg_vecs, wide, &vpt, &threads))
            return fail(GPUK_ERR_UNSUPPORTED, "row of %d vectors is longer than the largest tile", row_vecs);
        if (!fused) { vpt = 4; threads = std::max(32, ((row_vecs + 3) / 4 + 31) / 32 * 32); }
    }
    int per_sm = std::max(1, std::min(4, 1024 / threads));
    if (ctas_per_sm_limit > 0) per_sm = std::min(per_sm, ctas_per_sm_limit);
    const int64_t cta_cap = std::min<int64_t>(static_cast<int64_t>(sm_count) * per_sm, kMaxBlocks);
    int rpc = 1;
    if (world_size > 1 && !one_shot) {
        const int vpr = (row_vecs + world_size - 1) / world_size;
        if (rows > cta_cap) rpc = std::max(1, std::min(4, (threads + vpr - 1) / vpr));
        if (ov.rows_per_chunk > 0) rpc = std::min(ov.rows_per_chunk, 64);
    }
    const int64_t nchunks = (rows + rpc - 1) / rpc;
    int64_t grid;
    if (world_size == 1) grid = std::min<int64_t>(rows, static_cast<int64_t>(sm_count) * 8);
    else grid = std::min<int64_t>(nchunks, cta_cap / cluster) * cluster;
    // two-shot without clusters: the warp-specialised kernel, one CTA per SM
    out->ws = 0;
    out->ws_vpt = out->ws_tf = out->ws_tr = out->ws_ts = out->ws_grid = 0;
    if (world_size > 1 && !one_shot && cluster == 1 && ov.allow_ws) {
        int wv = fused ? 1 : 2;   // the plain all-reduce is built for the 2-vector tile only
        const int tf_max = ov.ws_tf > 0 && fused ? ov.ws_tf : kWsFinishThreads;
        while (wv < 8 && (row_vecs + wv - 1) / wv > tf_max) wv *= 2;
        const int tf = ((row_vecs + wv - 1) / wv + 31) / 32 * 32;
        const int tr = ov.ws_tr > 0 ? ov.ws_tr : kWsReduceThreads, tsc = ov.ws_ts > 0 ? ov.ws_ts : kWsScatterThreads;
        if (tf <= tf_max && tf + tr + tsc <= kWsMaxThreads) {
            out->ws = 1;
            out->ws_vpt = wv;
            out->ws_tf = tf;
            out->ws_tr = tr;
            out->ws_ts = tsc;
            out->ws_grid = static_cast<int>(std::min<int64_t>(rows, sm_count));
        }
    }
    out->cluster = cluster;
    out->lead_push = kDefaultLeadPush;
    out->lead_reduce = kDefaultLeadReduce;
    out->one_shot = one_shot ? 1 : 0;
    out->vpt = vpt;
    out->threads = threads;
    out->rows_per_chunk = rpc;
    out->grid = static_cast<int>(std::max<int64_t>(grid, 0));
    out->rows = static_cast<int>(rows);
    out->row_vecs = row_vecs;
    out->message_bytes = bytes;
    return GPUK_OK;
}

// ---------------------------------------------------------------------------------------
// workspace
// ---------------------------------------------------------------------------------------
int gpuk_ws_create(int device_id, int rank, int world_size, int64_t max_size_in_bytes,
                   int64_t comm_ptrs_buf_len, gpuk_ws **out) {
    (void)comm_ptrs_buf_len;
    if (!out) return fail(GPUK_ERR_INVALID_ARGUMENT, "ws_create: out is null");
    *out = nullptr;
    if (!valid_world(world_size)) return fail(GPUK_ERR_INVALID_ARGUMENT, "world size is not supported");
    if (rank < 0 || rank >= world_size) return fail(GPUK_ERR_INVALID_ARGUMENT, "invalid rank passed in");
    if (max_size_in_bytes <= 0) return fail(GPUK_ERR_INVALID_ARGUMENT, "max_size_in_bytes must be positive");
    if (device_id < 0) return fail(GPUK_ERR_INVALID_ARGUMENT, "invalid device id");
    GPUK_CUDA(cudaSetDevice(device_id));
    gpuk_ws *ws = new (std::nothrow) gpuk_ws();
    if (!ws) return fail(GPUK_ERR_CUDA, "out of host memory");
    ws->device = device_id;
    ws->rank = rank;
    ws->world = world_size;
    int sms = 0;
    if (cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, device_id) == cudaSuccess && sms > 0) ws->sm_count = sms;
    const int64_t align = 256ll * world_size;
    ws->cap = (max_size_in_bytes + align - 1) / align * align;
    ws->rs_slot_bytes = ws->cap / world_size + kRsSlack;
    ws->ag_off = ws->rs_slot_bytes * world_size;
    ws->ts_stride = ws->ag_off + ws->cap;
    ws->os_off = 2 * ws->ts_stride;
    ws->os_slot_bytes = std::min<int64_t>(ws->cap, kOneShotSlotBytes);
    ws->data_bytes = ws->os_off + 2 * world_size * ws->os_slot_bytes + kTailBytes;
    cudaError_t e = cudaMalloc(&ws->data, ws->data_bytes);
    if (e == cudaSuccess) e = fill_empty(ws->data, ws->data_bytes);
    if (e == cudaSuccess) e = cudaMalloc(&ws->flags, kFlagBytes);
    if (e == cudaSuccess) e = cudaMalloc(&ws->st, sizeof(LocalState));
    if (e == cudaSuccess) e = cudaMemset(ws->flags, 0, kFlagBytes);
    if (e == cudaSuccess) {
        LocalState init;
        memset(&init, 0, sizeof(init));
        init.timeout_ns = kDefaultTimeoutNs;
        e = cudaMemcpy(ws->st, &init, sizeof(init), cudaMemcpyHostToDevice);
    }
    if (e != cudaSuccess) {
        cudaFree(ws->data);
        cudaFree(ws->flags);
        cudaFree(ws->st);
        delete ws;
        return fail(GPUK_ERR_CUDA, "workspace allocation failed: %s", cudaGetErrorString(e));
    }
    ws->peer_data[rank] = ws->data;
    ws->peer_flags[rank] = ws->flags;
    *out = ws;
    return GPUK_OK;
}

int gpuk_ws_destroy(gpuk_ws *ws) {
    if (!ws) return GPUK_OK;
    cudaSetDevice(ws->device);
    cudaDeviceSynchronize();
    for (void *p : ws->ipc_opened) cudaIpcCloseMemHandle(p);
    cudaFree(ws->data);
    cudaFree(ws->flags);
    cudaFree(ws->st);
    cudaFree(ws->emul_params);
    delete ws;
    return GPUK_OK;
}

static int export_handle(gpuk_ws *ws, void *ptr, uint8_t *out) {
    if (!ws || !out) return fail(GPUK_ERR_INVALID_ARGUMENT, "null workspace or output");
    static_assert(sizeof(cudaIpcMemHandle_t) == GPUK_IPC_HANDLE_BYTES, "IPC handle size");
    GPUK_CUDA(cudaSetDevice(ws->device));
    cudaIpcMemHandle_t h;
    GPUK_CUDA(cudaIpcGetMemHandle(&h, ptr));
    memcpy(out, &h, sizeof(h));
    return GPUK_OK;
}

int gpuk_ws_get_barrier_handle(gpuk_ws *ws, uint8_t out[GPUK_IPC_HANDLE_BYTES]) {
    return export_handle(ws, ws ? ws->flags : nullptr, out);
}
int gpuk_ws_get_data_handle(gpuk_ws *ws, uint8_t out[GPUK_IPC_HANDLE_BYTES]) {
    return export_handle(ws, ws ? ws->data : nullptr, out);
}

static int open_handles(gpuk_ws *ws, const uint8_t *handles, int n, void **table, bool *ready) {
    if (!ws || !handles) return fail(GPUK_ERR_INVALID_ARGUMENT, "null workspace or handles");
    if (n != ws->world) return fail(GPUK_ERR_INVALID_ARGUMENT, "expected %d handles, got %d", ws->world, n);
    GPUK_CUDA(cudaSetDevice(ws->device));
    for (int r = 0; r < n; ++r) {
        if (r == ws->rank) continue;
        cudaIpcMemHandle_t h;
        memcpy(&h, handles + static_cast<size_t>(r) * GPUK_IPC_HANDLE_BYTES, sizeof(h));
        void *p = nullptr;
        cudaError_t e = cudaIpcOpenMemHandle(&p, h, cudaIpcMemLazyEnablePeerAccess);
        if (e != cudaSuccess) {
            cudaGetLastError();
            return fail(GPUK_ERR_CUDA, "cudaIpcOpenMemHandle for rank %d failed: %s", r, cudaGetErrorString(e));
        }
        table[r] = p;
        ws->ipc_opened.push_back(p);
    }
    *ready = true;
    return GPUK_OK;
}

int gpuk_ws_open_barrier_handles(gpuk_ws *ws, const uint8_t *handles, int n) {
    return open_handles(ws, handles, n, ws ? ws->peer_flags : nullptr, ws ? &ws->have_flags : nullptr);
}
int gpuk_ws_open_data_handles(gpuk_ws *ws, const uint8_t *handles, int n) {
    return open_handles(ws, handles, n, ws ? ws->peer_data : nullptr, ws ? &ws->have_data : nullptr);
}

int gpuk_ws_local_pointers(gpuk_ws *ws, void **flags, void **data) {
    if (!ws || !flags || !data) return fail(GPUK_ERR_INVALID_ARGUMENT, "null argument");
    *flags = ws->flags;
    *data = ws->data;
    return GPUK_OK;
}

int gpuk_ws_set_peer_pointers(gpuk_ws *ws, void *const *flags, void *const *data, int n) {
    if (!ws || !flags || !data) return fail(GPUK_ERR_INVALID_ARGUMENT, "null argument");
    if (n != ws->world) return fail(GPUK_ERR_INVALID_ARGUMENT, "expected %d pointers, got %d", ws->world, n);
    for (int r = 0; r < n; ++r) {
        if (!flags[r] || !data[r]) return fail(GPUK_ERR_INVALID_ARGUMENT, "null peer pointer for rank %d", r);
        if (r == ws->rank) continue;
        ws->peer_flags[r] = flags[r];
        ws->peer_data[r] = data[r];
    }
    ws->have_flags = ws->have_data = true;
    return GPUK_OK;
}

int gpuk_ws_attach_symmetric(gpuk_ws *ws, void *const *bases, int n, void *mc_base, int64_t bytes) {
    if (!ws || !bases) return fail(GPUK_ERR_INVALID_ARGUMENT, "null workspace or buffer table");
    if (n != ws->world) return fail(GPUK_ERR_INVALID_ARGUMENT, "expected %d buffers, got %d", ws->world, n);
    if (bytes < kSymFlagBytes + 512) return fail(GPUK_ERR_INVALID_ARGUMENT, "symmetric buffer of %lld bytes is too small", (long long)bytes);
    for (int r = 0; r < n; ++r)
        if (!bases[r] || (reinterpret_cast<uintptr_t>(bases[r]) & 255u))
            return fail(GPUK_ERR_INVALID_ARGUMENT, "symmetric buffer of rank %d is null or not 256-byte aligned", r);
    if (reinterpret_cast<uintptr_t>(mc_base) & 255u) return fail(GPUK_ERR_INVALID_ARGUMENT, "multicast mapping is not 256-byte aligned");
    for (int r = 0; r < n; ++r) ws->sym[r] = static_cast<char *>(bases[r]);
    ws->sym_mc = static_cast<char *>(mc_base);
    ws->sym_cap = (bytes - kSymFlagBytes) / 2 / 256 * 256;
    ws->sym_flag_off = 2 * ws->sym_cap;
    return GPUK_OK;
}

int gpuk_enable_peer_access(int n_devices) {
    int count = 0;
    GPUK_CUDA(cudaGetDeviceCount(&count));
    if (n_devices <= 0 || n_devices > count) return fail(GPUK_ERR_INVALID_ARGUMENT, "%d devices requested, %d present", n_devices, count);
    int prev = 0;
    GPUK_CUDA(cudaGetDevice(&prev));
    for (int a = 0; a < n_devices; ++a) {
        GPUK_CUDA(cudaSetDevice(a));
        for (int b = 0; b < n_devices; ++b) {
            if (a == b) continue;
            int can = 0;
            GPUK_CUDA(cudaDeviceCanAccessPeer(&can, a, b));
            if (!can) return fail(GPUK_ERR_UNSUPPORTED, "device %d cannot access device %d", a, b);
            cudaError_t e = cudaDeviceEnablePeerAccess(b, 0);
            if (e == cudaErrorPeerAccessAlreadyEnabled) cudaGetLastError();
            else if (e != cudaSuccess) return fail(GPUK_ERR_CUDA, "cudaDeviceEnablePeerAccess(%d->%d): %s", a, b, cudaGetErrorString(e));
        }
    }
    GPUK_CUDA(cudaSetDevice(prev));
    return GPUK_OK;
}

// ---- capture-registration surface: nothing to register in a push design ------------------
int gpuk_ws_capture_clear(gpuk_ws *ws) {
    if (!ws) return fail(GPUK_ERR_INVALID_ARGUMENT, "null workspace");
    return GPUK_OK;
}
int gpuk_ws_captured_count(gpuk_ws *ws, int *count) {
    if (!ws || !count) return fail(GPUK_ERR_INVALID_ARGUMENT, "null argument");
    *count = 0;
    return GPUK_OK;
}
int gpuk_ws_open_captured_handles(gpuk_ws *ws, const uint8_t *handles, const int64_t *offsets, int n, int64_t ptr_idx) {
    (void)handles; (void)offsets; (void)n;
    if (!ws) return fail(GPUK_ERR_INVALID_ARGUMENT, "null workspace");
    return fail(GPUK_ERR_INVALID_ARGUMENT, "no captured tensor with index %lld: captured calls need no registration", (long long)ptr_idx);
}

static int base_of(const void *ptr, void **base) {
    if (!ptr) return fail(GPUK_ERR_INVALID_ARGUMENT, "null pointer");
    // the driver entry point is looked up at run time so that this library loads without libcuda
    typedef CUresult (*PointerGetAttribute)(void *, CUpointer_attribute, CUdeviceptr);
    static PointerGetAttribute get_attr = nullptr;
    if (!get_attr) {
        void *fn = nullptr;
        cudaDriverEntryPointQueryResult qr;
        cudaError_t e = cudaGetDriverEntryPoint("cuPointerGetAttribute", &fn, cudaEnableDefault, &qr);
        if (e != cudaSuccess || !fn) {
            cudaGetLastError();
            return fail(GPUK_ERR_CUDA, "cuPointerGetAttribute is not available");
        }
        get_attr = reinterpret_cast<PointerGetAttribute>(fn);
    }
    CUdeviceptr b = 0;
    CUresult r = get_attr(&b, CU_POINTER_ATTRIBUTE_RANGE_START_ADDR, reinterpret_cast<CUdeviceptr>(ptr));
    if (r != CUDA_SUCCESS) return fail(GPUK_ERR_CUDA, "failed to get pointer attr");
    *base = reinterpret_cast<void *>(b);
    return GPUK_OK;
}
int gpuk_tensor_ipc_handle(const void *ptr, uint8_t out[GPUK_IPC_HANDLE_BYTES]) {
    if (!out) return fail(GPUK_ERR_INVALID_ARGUMENT, "null output");
    void *base = nullptr;
    int rc = base_of(ptr, &base);
    if (rc) return rc;
    cudaIpcMemHandle_t h;
    GPUK_CUDA(cudaIpcGetMemHandle(&h, base));
    memcpy(out, &h, sizeof(h));
    return GPUK_OK;
}
int gpuk_tensor_ipc_offset(const void *ptr, int64_t *offset) {
    if (!offset) return fail(GPUK_ERR_INVALID_ARGUMENT, "null output");
    void *base = nullptr;
    int rc = base_of(ptr, &base);
    if (rc) return rc;
    *offset = reinterpret_cast<const char *>(ptr) - reinterpret_cast<const char *>(base);
    return GPUK_OK;
}

// ---- knobs and status --------------------------------------------------------------------
int gpuk_ws_set_oneshot_max_bytes(gpuk_ws *ws, int64_t bytes) {
    if (!ws) return fail(GPUK_ERR_INVALID_ARGUMENT, "null workspace");
    ws->oneshot_max_bytes = bytes > 0 ? bytes : 0;
    return GPUK_OK;
}
int gpuk_ws_set_option(gpuk_ws *ws, const char *name, int64_t value) {
    if (!ws || !name) return fail(GPUK_ERR_INVALID_ARGUMENT, "null workspace or option name");
    const std::string n(name);
    if (n == "rows_per_chunk") {
        if (value < 0 || value > 64) return fail(GPUK_ERR_INVALID_ARGUMENT, "rows_per_chunk must be in [0, 64]");
        ws->opt_rows_per_chunk = static_cast<int>(value);
    } else if (n == "ctas_per_sm") {
        if (value < 0 || value > 16) return fail(GPUK_ERR_INVALID_ARGUMENT, "ctas_per_sm must be in [0, 16]");
        ws->opt_ctas_per_sm = static_cast<int>(value);
    } else if (n == "lead_push" || n == "lead_reduce") {
        if (value < 0 || value > (1 << 20)) return fail(GPUK_ERR_INVALID_ARGUMENT, "%s must be in [0, 2^20]", name);
        (n == "lead_push" ? ws->opt_lead_push : ws->opt_lead_reduce) = static_cast<int>(value);
    } else if (n == "cluster") {
        if (value != 0 && value != 1 && value != 2 && value != 4 && value != 8) return fail(GPUK_ERR_INVALID_ARGUMENT, "cluster must be 0, 1, 2, 4 or 8");
        ws->opt_cluster = static_cast<int>(value);
    } else if (n == "two_shot_ws") {
        if (value != 0 && value != 1) return fail(GPUK_ERR_INVALID_ARGUMENT, "two_shot_ws must be 0 or 1");
        ws->opt_two_shot_ws = static_cast<int>(value);
    } else if (n == "two_rank_one_hop") {
        if (value != 0 && value != 1) return fail(GPUK_ERR_INVALID_ARGUMENT, "two_rank_one_hop must be 0 or 1");
        ws->opt_two_rank_one_hop = static_cast<int>(value);
    } else if (n == "ws_finish_threads" || n == "ws_reduce_threads" || n == "ws_scatter_threads") {
        if (value < 0 || value > 512 || value % 32) return fail(GPUK_ERR_INVALID_ARGUMENT, "%s must be a multiple of 32 in [0, 512]", name);
        (n == "ws_finish_threads" ? ws->opt_ws_tf : (n == "ws_reduce_threads" ? ws->opt_ws_tr : ws->opt_ws_ts)) = static_cast<int>(value);
    } else if (n == "ws_max_ctas") {
        if (value < 0 || value > kMaxBlocks) return fail(GPUK_ERR_INVALID_ARGUMENT, "ws_max_ctas must be in [0, %d]", kMaxBlocks);
        ws->opt_ws_max_ctas = static_cast<int>(value);
    } else if (n == "ws_scatter_lead") {
        if (value < -1 || value > (1 << 20)) return fail(GPUK_ERR_INVALID_ARGUMENT, "ws_scatter_lead must be in [-1, 2^20]");
        ws->opt_ws_scatter_lead = static_cast<int>(value);
    } else if (n == "test_withhold_cluster") {
        ws->test_withhold_cluster = value != 0;
    } else if (n == "gather_multicast") {
        if (value != 0 && value != 1) return fail(GPUK_ERR_INVALID_ARGUMENT, "gather_multicast must be 0 or 1");
        if (value && (!ws->sym[ws->rank] || !ws->sym_mc))
            return fail(GPUK_ERR_NOT_READY, "gather_multicast needs symmetric memory with a multicast mapping (gpuk_ws_attach_symmetric)");
        if (value) {
            // the two halves of the symmetric buffer become the gather areas of the two call parities: at rest
            GPUK_CUDA(cudaSetDevice(ws->device));
            GPUK_CUDA(cudaDeviceSynchronize());
            GPUK_CUDA(fill_empty(ws->sym[ws->rank], 2 * ws->sym_cap));
        }
        ws->gather_multicast = value != 0;
    } else if (n == "sym_multicast") {
        if (value != 0 && value != 1) return fail(GPUK_ERR_INVALID_ARGUMENT, "sym_multicast must be 0 or 1");
        ws->sym_use_mc = value != 0;
    } else if (n == "sym_min_bytes") {
        if (value < 0) return fail(GPUK_ERR_INVALID_ARGUMENT, "sym_min_bytes must not be negative");
        ws->sym_min_bytes = value;
    } else if (n == "oneshot_max_bytes") {
        return gpuk_ws_set_oneshot_max_bytes(ws, value);
    } else {
        return fail(GPUK_ERR_INVALID_ARGUMENT, "unknown option '%s'", name);
    }
    return GPUK_OK;
}
int gpuk_ws_set_ready_words(gpuk_ws *ws, const uint32_t *ready, int rows_per_word, uint32_t value) {
    if (!ws) return fail(GPUK_ERR_INVALID_ARGUMENT, "null workspace");
    if (ready && rows_per_word <= 0) return fail(GPUK_ERR_INVALID_ARGUMENT, "rows_per_word must be positive");
    if (ready && (reinterpret_cast<uintptr_t>(ready) & 3u)) return fail(GPUK_ERR_INVALID_ARGUMENT, "ready words must be 4-byte aligned");
    ws->ready = ready;
    ws->ready_rows = ready ? rows_per_word : 0;
    ws->ready_value = value;
    return GPUK_OK;
}
int gpuk_ws_set_timeout_ns(gpuk_ws *ws, uint64_t ns) {
    if (!ws || ns == 0) return fail(GPUK_ERR_INVALID_ARGUMENT, "null workspace or zero budget");
    GPUK_CUDA(cudaSetDevice(ws->device));
    unsigned long long v = ns;
    GPUK_CUDA(cudaMemcpy(&ws->st->timeout_ns, &v, sizeof(v), cudaMemcpyHostToDevice));
    return GPUK_OK;
}
int gpuk_ws_status(gpuk_ws *ws, uint32_t out[8]) {
    if (!ws || !out) return fail(GPUK_ERR_INVALID_ARGUMENT, "null argument");
    GPUK_CUDA(cudaSetDevice(ws->device));
    GPUK_CUDA(cudaDeviceSynchronize());
    LocalState host;
    GPUK_CUDA(cudaMemcpy(&host, ws->st, sizeof(host), cudaMemcpyDeviceToHost));
    memcpy(out, host.status, sizeof(host.status));
    if (out[0] == kStatusClusterMismatch)
        return fail(GPUK_ERR_BAD_LAUNCH, "rank %u CTA %u ran in a thread-block cluster of %u CTAs, not the planned size; nothing was written",
                    out[1], out[2], out[6]);
    if (out[0] != 0)
        return fail(GPUK_ERR_PEER_TIMEOUT, "rank %u CTA %u thread %u gave up waiting for data from rank %u in stage %u (word seen 0x%08x)",
                    out[1], out[2], out[5], out[4], out[3], out[6]);
    return GPUK_OK;
}
int gpuk_ws_clear_status(gpuk_ws *ws) {
    if (!ws) return fail(GPUK_ERR_INVALID_ARGUMENT, "null workspace");
    GPUK_CUDA(cudaSetDevice(ws->device));
    GPUK_CUDA(cudaDeviceSynchronize());
    GPUK_CUDA(cudaMemset(ws->st->status, 0, sizeof(uint32_t) * kStatusWords));
    GPUK_CUDA(cudaMemset(&ws->st->abort, 0, sizeof(uint32_t)));
    // an exchange that gave up may have left vectors unconsumed: put the staging back to rest
    GPUK_CUDA(fill_empty(ws->data, ws->data_bytes));
    if (ws->gather_multicast && ws->sym[ws->rank]) GPUK_CUDA(fill_empty(ws->sym[ws->rank], 2 * ws->sym_cap));
    return GPUK_OK;
}

}  // extern "C"

// ---------------------------------------------------------------------------------------
// kernels launched from this file
// ---------------------------------------------------------------------------------------
namespace {

__global__ void selftest_wait_kernel(LocalState *st, const uint4 *vec, int rank) {
    if (threadIdx.x == 0) wait_landed(vec, ld_poll(vec), st, rank, kStageSelfTest, rank);
}

template <typename F>
int by_dtype(int dtype, F &&f) {
    switch (dtype) {
    case GPUK_DTYPE_BF16: return f(static_cast<__nv_bfloat16 *>(nullptr));
    case GPUK_DTYPE_F16: return f(static_cast<__half *>(nullptr));
    case GPUK_DTYPE_F32: return f(static_cast<float *>(nullptr));
    default: return fail(GPUK_ERR_UNSUPPORTED, "unknown dtype %d", dtype);
    }
}

struct CallArgs {
    const void *in;
    const void *residual;
    const void *gamma;
    void *residual_out;
    void *norm_out;
    float *scale_out;
    int64_t numel;
    int hidden;      // 0: plain all-reduce (in place over `in`)
    int dtype;
    float eps;
    int quant_type;
};

int check_fused_args(const CallArgs &a, Quant *q) {
    if (!quant_from_type(a.quant_type, q)) return fail(GPUK_ERR_INVALID_ARGUMENT, "unknown quant_type %d", a.quant_type);
    if (!a.in || !a.residual || !a.gamma || !a.residual_out || !a.norm_out)
        return fail(GPUK_ERR_INVALID_ARGUMENT, "null tensor pointer");
    if (q->mode != kQuantNone && !a.scale_out) return fail(GPUK_ERR_INVALID_ARGUMENT, "scale_out is null");
    if (!aligned16(a.in) || !aligned16(a.residual) || !aligned16(a.gamma) || !aligned16(a.residual_out) || !aligned16(a.norm_out))
        return fail(GPUK_ERR_INVALID_ARGUMENT, "tensor pointers must be 16-byte aligned");
    if (a.hidden <= 0) return fail(GPUK_ERR_INVALID_ARGUMENT, "hidden must be positive");
    return GPUK_OK;
}

void fill_epilogue(const CallArgs &a, const Quant &q, int row_vecs, EpilogueArgs *ep) {
    ep->residual = a.residual;
    ep->gamma = a.gamma;
    ep->residual_out = a.residual_out;
    ep->norm_out = a.norm_out;
    ep->scale_out = a.scale_out;
    ep->hidden = a.hidden;
    ep->row_vecs = row_vecs;
    ep->eps = a.eps;
    ep->hidden_f = static_cast<float>(a.hidden);
    ep->inv_hidden = static_cast<float>(1.0 / static_cast<double>(a.hidden));
    ep->q = q;
}

// Fills the parameter block of one rank and the launch shape shared by all ranks.
int build_ar_call(gpuk_ws *ws, const CallArgs &a, int force_mode, bool emulated, ArParams *p, ArShape *shape) {
    if (!ws->have_data || !ws->have_flags) return fail(GPUK_ERR_NOT_READY, "peer handles have not been opened");
    const bool fused = a.hidden > 0;
    Quant q = make_quant(kQuantNone, 0, 0.f);
    if (fused) {
        int rc = check_fused_args(a, &q);
        if (rc) return rc;
    } else {
        if (!a.in) return fail(GPUK_ERR_INVALID_ARGUMENT, "null tensor pointer");
        if (!aligned16(a.in)) return fail(GPUK_ERR_INVALID_ARGUMENT, "tensor pointers must be 16-byte aligned");
    }
    gpuk_plan plan;
    PlanOverrides ov;
    ov.cluster = ws->opt_cluster;
    ov.allow_ws = ws->opt_two_shot_ws != 0;
    ov.ws_tf = ws->opt_ws_tf;
    ov.ws_tr = ws->opt_ws_tr;
    ov.ws_ts = ws->opt_ws_ts;
    int rc = plan_call(ws->world, a.numel, a.hidden, a.dtype, ws->sm_count, 0, ws->oneshot_max_bytes, ov, &plan);
    if (rc) return rc;
    if (plan.message_bytes > ws->cap)
        return fail(GPUK_ERR_TOO_LARGE, "message of %lld bytes exceeds the workspace (%lld bytes)",
                    (long long)plan.message_bytes, (long long)ws->cap);
    bool one_shot = plan.one_shot != 0;
    int sym = 0;
    if (force_mode == GPUK_MODE_SYMMETRIC ||
        (force_mode == GPUK_MODE_AUTO && fused && !one_shot && ws->sym[ws->rank] && ws->sym_min_bytes > 0 && !ws->gather_multicast &&
         plan.message_bytes >= ws->sym_min_bytes && plan.message_bytes <= ws->sym_cap)) {
        if (!fused) return fail(GPUK_ERR_UNSUPPORTED, "the exchange through symmetric memory is built for the fused operator only");
        if (ws->gather_multicast)
            return fail(GPUK_ERR_UNSUPPORTED, "the symmetric buffer holds the gather areas (option gather_multicast): the exchange through symmetric memory is off");
        if (!ws->sym[ws->rank]) return fail(GPUK_ERR_NOT_READY, "no symmetric memory attached to this workspace");
        if (plan.message_bytes > ws->sym_cap)
            return fail(GPUK_ERR_TOO_LARGE, "message of %lld bytes exceeds the symmetric buffer (%lld bytes per message)",
                        (long long)plan.message_bytes, (long long)ws->sym_cap);
        sym = (ws->sym_mc && ws->sym_use_mc && !emulated) ? 2 : 1;
        force_mode = GPUK_MODE_TWO_SHOT;
        ov.allow_cluster = false;
        rc = plan_call(ws->world, a.numel, a.hidden, a.dtype, ws->sm_count, 0, 1, ov, &plan);
        if (rc) return rc;
        one_shot = false;
    }
    if (force_mode == 1) {
        if (plan.message_bytes > ws->os_slot_bytes || plan.rows > kMaxBlocks)
            return fail(GPUK_ERR_TOO_LARGE, "message too large for the one-shot path");
        one_shot = true;
    } else if (force_mode == 2) {
        one_shot = false;
    }
    if (one_shot != (plan.one_shot != 0)) {
        // re-plan with the crossover forced to the requested side
        rc = plan_call(ws->world, a.numel, a.hidden, a.dtype, ws->sm_count, 0, one_shot ? kOneShotSlotBytes : 1, ov, &plan);
        if (rc) return rc;
        if ((plan.one_shot != 0) != one_shot) return fail(GPUK_ERR_UNSUPPORTED, "requested exchange mode is not available for this shape");
    }
    const bool use_ws = plan.ws != 0 && !one_shot && !sym;
    if (!one_shot && !use_ws && ws->opt_rows_per_chunk > 0) plan.rows_per_chunk = std::min(ws->opt_rows_per_chunk, 64);
    if (ws->opt_ctas_per_sm > 0) plan.grid = std::min<int64_t>(plan.grid, static_cast<int64_t>(ws->sm_count) * ws->opt_ctas_per_sm);
    const int es = elem_size(a.dtype);
    memset(p, 0, sizeof(*p));
    p->in = a.in;
    p->out = const_cast<void *>(a.in);
    p->total_vecs = a.numel * es / 16;
    p->rows = plan.rows;
    p->row_vecs = plan.row_vecs;
    p->rows_per_chunk = plan.rows_per_chunk;
    p->seg_vecs = (plan.row_vecs + plan.cluster - 1) / plan.cluster;
    p->cluster = plan.cluster;
    if (ws->ready && !use_ws)
        return fail(GPUK_ERR_UNSUPPORTED, "ready words need the two-shot exchange with specialised warps, which this call does not take "
                                          "(message too small, rows shared by clusters, or switched off): order the call behind the producer instead");
    if (use_ws) {
        plan.grid = ws->opt_ws_max_ctas > 0 ? std::min(plan.ws_grid, ws->opt_ws_max_ctas) : plan.ws_grid;
        p->ready = ws->ready;
        p->ready_rows = ws->ready_rows;
        p->ready_value = ws->ready_value;
        plan.rows_per_chunk = 1;
        p->rows_per_chunk = 1;
        // rows the scatter may run ahead of the finish.  Measured at eight ranks with the multicast gather, 2 / 8 rows:
        // 16 MiB (7 rows per CTA) 59.2 / 61.5 us, 224 MiB (111 rows per CTA) 681 / 663 us; two ranks, 224 MiB: 439 / 407 us.
        const int64_t rows_per_cta = (plan.rows + plan.ws_grid - 1) / std::max(plan.ws_grid, 1);
        p->scatter_lead = ws->opt_ws_scatter_lead < 0 ? (rows_per_cta >= 32 ? kWsScatterLeadLong : kWsScatterLeadShort) : ws->opt_ws_scatter_lead;
        // gather areas: in the workspace, or in symmetric memory behind the NVSwitch multicast address
        const bool mc = ws->gather_multicast && ws->sym_mc && !emulated && plan.message_bytes <= ws->sym_cap;
        for (int r = 0; r < ws->world; ++r)
            p->ag_base[r] = mc ? ws->sym[r] : static_cast<char *>(ws->peer_data[r]) + ws->ag_off;
        p->ag_stride = mc ? ws->sym_cap : ws->ts_stride;
        p->ag_mc = mc ? ws->sym_mc : nullptr;
        p->tf = plan.ws_tf;
        p->tr = plan.ws_tr;
        p->ts = plan.ws_ts;
        // no bounds checks in the finishing warps when every row, the last included, fills the tile
        p->full = (plan.row_vecs == plan.ws_vpt * plan.ws_tf && p->total_vecs % plan.row_vecs == 0) ? 1 : 0;
        // Two ranks: whole rows straight into the peer's gather area, one hop.  The finishing warps then read this
        // rank's input themselves, so the outputs must not overlap it (a finished row would overwrite input that has
        // not been pushed yet), and an input still in the making (ready words) keeps the two-hop exchange, whose
        // finishing warps never touch the input.
        auto overlaps_in = [&](const void *o, int64_t bytes) {
            const char *b = static_cast<const char *>(o), *i0 = static_cast<const char *>(a.in);
            return o && b < i0 + plan.message_bytes && i0 < b + bytes;
        };
        // exact sizes: two live tensors that merely lie next to each other must not count, or ranks whose allocators
        // placed them differently would pick different kernels (aliasing on purpose is the same on every rank)
        const int64_t norm_bytes = q.mode == kQuantNone ? plan.message_bytes : a.numel;
        p->one_hop = (ws->world == 2 && fused && ws->opt_two_rank_one_hop && !ws->ready &&
                      !overlaps_in(a.residual_out, plan.message_bytes) && !overlaps_in(a.norm_out, norm_bytes)) ? 1 : 0;
        if (p->one_hop) p->ts = kWs1PushThreads, p->tr = 0;
    }
    p->lead_push = std::max(1, ws->opt_lead_push > 0 ? ws->opt_lead_push : plan.lead_push);
    p->lead_reduce = std::max(1, ws->opt_lead_reduce > 0 ? ws->opt_lead_reduce : plan.lead_reduce);
    if (fused) fill_epilogue(a, q, plan.row_vecs, &p->ep);
    p->rank = ws->rank;
    p->vpr = (plan.row_vecs + ws->world - 1) / ws->world;
    for (int r = 0; r < ws->world; ++r) {
        p->peer_data[r] = static_cast<char *>(ws->peer_data[r]);
    }
    p->st = ws->st;
    p->rs_slot_bytes = ws->rs_slot_bytes;
    p->ag_off = ws->ag_off;
    p->ts_stride = ws->ts_stride;
    p->os_off = ws->os_off;
    p->os_slot_bytes = ws->os_slot_bytes;
    for (int r = 0; r < ws->world; ++r) p->sym[r] = ws->sym[r];
    p->sym_mc = ws->sym_mc;
    p->sym_in_off = 0;
    p->sym_out_off = ws->sym_cap;
    p->sym_flag_off = ws->sym_flag_off;
    if (!one_shot && !sym && static_cast<int64_t>(plan.rows) * p->vpr * 16 > ws->rs_slot_bytes)
        return fail(GPUK_ERR_TOO_LARGE, "message does not fit the reduce-scatter slots of the workspace");

    shape->world = ws->world;
    shape->vpt = use_ws ? plan.ws_vpt : plan.vpt;
    shape->two_shot = !one_shot;
    shape->fused = fused;
    shape->ws = use_ws ? (p->one_hop ? 2 : 1) : 0;
    shape->threads = use_ws ? p->tf + p->tr + p->ts : plan.threads;
    shape->cluster = plan.cluster;
    shape->grid = plan.grid;
    shape->sym = sym;
    // the grid must be co-resident: CTAs of equal index on different ranks wait for each other
    const uint32_t key = static_cast<uint32_t>(a.dtype) | (shape->vpt << 4) | (one_shot ? 1u << 8 : 0u) |
                         (fused ? 1u << 9 : 0u) | (emulated ? 1u << 10 : 0u) | (use_ws ? 1u << 11 : 0u) | (p->one_hop ? 1u << 30 : 0u) |
                         (static_cast<uint32_t>(shape->threads) << 12) |
                         (static_cast<uint32_t>(plan.cluster) << 24) | (static_cast<uint32_t>(sym) << 28);
    int64_t resident = 0;
    auto cached = ws->occupancy.find(key);
    if (cached != ws->occupancy.end()) {
        resident = cached->second;
    } else {
        rc = by_dtype(a.dtype, [&](auto *t) {
            using T = std::remove_pointer_t<decltype(t)>;
            cudaError_t e = ar_resident_ctas<T>(*shape, emulated, ws->sm_count, &resident);
            if (e != cudaSuccess || resident <= 0) {
                cudaGetLastError();
                return fail(GPUK_ERR_CUDA, "occupancy query failed for the selected kernel: %s", cudaGetErrorString(e));
            }
            return static_cast<int>(GPUK_OK);
        });
        if (rc) return rc;
        ws->occupancy[key] = resident;
    }
    if (emulated) resident = resident / ws->world / plan.cluster * plan.cluster;
    const int64_t nchunks = (static_cast<int64_t>(plan.rows) + plan.rows_per_chunk - 1) / plan.rows_per_chunk;
    int64_t clusters = std::min<int64_t>(std::min<int64_t>(plan.grid, resident) / plan.cluster, nchunks);
    if (clusters < 1) return fail(GPUK_ERR_UNSUPPORTED, "the GPU cannot hold one cluster of %d CTAs of the selected kernel", plan.cluster);
    shape->grid = static_cast<int>(clusters * plan.cluster);
    if (ws->test_withhold_cluster) shape->cluster = 1;   // the kernels must notice and report it
    return GPUK_OK;
}

}  // namespace

extern "C" {

int gpuk_ws_selftest_wait(gpuk_ws *ws, void *stream) {
    if (!ws) return fail(GPUK_ERR_INVALID_ARGUMENT, "null workspace");
    GPUK_CUDA(cudaSetDevice(ws->device));
    // the tail of the staging allocation is never written by any exchange
    const uint4 *vec = reinterpret_cast<const uint4 *>(ws->data + ws->data_bytes - kTailBytes);
    selftest_wait_kernel<<<1, 32, 0, static_cast<cudaStream_t>(stream)>>>(ws->st, vec, ws->rank);
    GPUK_CUDA(cudaGetLastError());
    return GPUK_OK;
}

int gpuk_residual_rms_quant(const void *in, const void *residual_in, const void *rms_gamma,
                            void *residual_out, void *norm_out, float *scale_out, int64_t numel,
                            int hidden, int dtype, float eps, int quant_type, void *stream) {
    CallArgs a = {in, residual_in, rms_gamma, residual_out, norm_out, scale_out, numel, hidden, dtype, eps, quant_type};
    Quant q;
    if (numel == 0) return GPUK_OK;
    int rc = check_fused_args(a, &q);
    if (rc) return rc;
    int device = 0, sms = kDefaultSmCount;
    GPUK_CUDA(cudaGetDevice(&device));
    cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, device);
    gpuk_plan plan;
    rc = gpuk_plan_allreduce_rms(1, numel, hidden, dtype, sms, 0, 0, &plan);
    if (rc) return rc;
    if (plan.rows == 0) return GPUK_OK;
    NormQuantParams p;
    memset(&p, 0, sizeof(p));
    p.in = in;
    p.rows = plan.rows;
    fill_epilogue(a, q, plan.row_vecs, &p.ep);
    // rows beyond one per resident CTA: persistent CTAs that stage rows through shared memory by bulk
    // copies, so that the next rows are in flight while the current one is reduced
    const int stages = g_tuning.k1_stages < 0 ? kDefaultK1Stages : g_tuning.k1_stages;
    const int64_t staged_min = g_tuning.k1_staged_min_rows < 0 ? kK1StagedMinRows(sms) : g_tuning.k1_staged_min_rows;
    const bool staged = stages >= 1 && plan.rows >= staged_min;
    return by_dtype(dtype, [&](auto *t) {
        using T = std::remove_pointer_t<decltype(t)>;
        cudaError_t e = cudaErrorInvalidConfiguration;
        if (staged) {
            // the persistent variant may use a wider CTA than the one-row-per-CTA kernel: fewer, faster row passes
            int vpt = plan.vpt, threads = plan.threads;
            const int want = g_tuning.k1_threads > 0 ? g_tuning.k1_threads : kDefaultK1Threads;
            while (vpt > 1 && threads * 2 <= want) { vpt /= 2; threads = ((plan.row_vecs + vpt - 1) / vpt + 31) / 32 * 32; }
            e = launch_norm_quant_staged<T>(p, vpt, threads, stages, sms, g_tuning.k1_ctas_per_sm, static_cast<cudaStream_t>(stream));
        }
        if (e == cudaErrorInvalidConfiguration) {
            if (staged) cudaGetLastError();
            e = launch_norm_quant<T>(p, plan.vpt, plan.threads, plan.grid, static_cast<cudaStream_t>(stream));
        }
        if (e != cudaSuccess) return fail(GPUK_ERR_CUDA, "kernel launch failed: %s", cudaGetErrorString(e));
        return static_cast<int>(GPUK_OK);
    });
}

int gpuk_set_tuning(const char *name, int64_t value) {
    if (!name) return fail(GPUK_ERR_INVALID_ARGUMENT, "null option name");
    const std::string n(name);
    if (n == "k1_stages") {
        if (value < -1 || value > 8) return fail(GPUK_ERR_INVALID_ARGUMENT, "k1_stages must be in [-1, 8]");
        g_tuning.k1_stages = static_cast<int>(value);
    } else if (n == "k1_threads") {
        if (value != 0 && value != 256 && value != 512 && value != 1024) return fail(GPUK_ERR_INVALID_ARGUMENT, "k1_threads must be 0, 256, 512 or 1024");
        g_tuning.k1_threads = static_cast<int>(value);
    } else if (n == "k1_staged_min_rows") {
        g_tuning.k1_staged_min_rows = value;
    } else if (n == "fp8_frags_per_warp") {
        if (value < 0 || value > 2) return fail(GPUK_ERR_INVALID_ARGUMENT, "fp8_frags_per_warp must be 0, 1 or 2");
        fp8_frags_per_warp_tuning = static_cast<int>(value);
    } else if (n == "k1_ctas_per_sm") {
        if (value < 0 || value > 8) return fail(GPUK_ERR_INVALID_ARGUMENT, "k1_ctas_per_sm must be in [0, 8]");
        g_tuning.k1_ctas_per_sm = static_cast<int>(value);
    } else {
        return fail(GPUK_ERR_INVALID_ARGUMENT, "unknown tuning option '%s'", name);
    }
    return GPUK_OK;
}

static int run_ar(gpuk_ws *ws, const CallArgs &a, void *stream) {
    if (!ws) return fail(GPUK_ERR_INVALID_ARGUMENT, "null workspace");
    if (a.numel == 0) return GPUK_OK;
    GPUK_CUDA(cudaSetDevice(ws->device));
    ArParams p;
    ArShape shape;
    int rc = build_ar_call(ws, a, 0, false, &p, &shape);
    ws->ready = nullptr;      // ready words apply to one call
    if (rc) return rc;
    return by_dtype(a.dtype, [&](auto *t) {
        using T = std::remove_pointer_t<decltype(t)>;
        cudaError_t e = launch_ar<T>(p, shape, static_cast<cudaStream_t>(stream));
        if (e != cudaSuccess) return fail(GPUK_ERR_CUDA, "kernel launch failed: %s", cudaGetErrorString(e));
        return static_cast<int>(GPUK_OK);
    });
}

int gpuk_allreduce_rms(gpuk_ws *ws, const void *allreduce_in, const void *residual_in,
                       const void *rms_gamma, void *residual_out, void *norm_out, float *scale_out,
                       int64_t numel, int hidden, int dtype, float eps, int quant_type, void *stream) {
    if (hidden <= 0) return fail(GPUK_ERR_INVALID_ARGUMENT, "hidden must be positive");
    CallArgs a = {allreduce_in, residual_in, rms_gamma, residual_out, norm_out, scale_out, numel, hidden, dtype, eps, quant_type};
    return run_ar(ws, a, stream);
}

int gpuk_allreduce_inplace(gpuk_ws *ws, void *data, int64_t numel, int dtype, void *stream) {
    CallArgs a = {data, nullptr, nullptr, nullptr, nullptr, nullptr, numel, 0, dtype, 0.f, 0};
    return run_ar(ws, a, stream);
}

int gpuk_emulated_allreduce_rms(gpuk_ws *const *wss, int world_size, void *const *allreduce_in,
                                const void *residual_in, const void *rms_gamma, void *const *residual_out,
                                void *const *norm_out, float *const *scale_out, int64_t numel, int hidden,
                                int dtype, float eps, int quant_type, int force_mode, void *stream) {
    if (!wss || !allreduce_in) return fail(GPUK_ERR_INVALID_ARGUMENT, "null argument");
    if (!valid_world(world_size)) return fail(GPUK_ERR_INVALID_ARGUMENT, "world size is not supported");
    if (numel == 0) return GPUK_OK;
    const bool fused = hidden > 0;
    if (fused && (!residual_out || !norm_out)) return fail(GPUK_ERR_INVALID_ARGUMENT, "null output arrays");
    ArParams host_params[kMaxRanks];
    ArShape shape = {};
    for (int r = 0; r < world_size; ++r) {
        gpuk_ws *ws = wss[r];
        if (!ws || ws->world != world_size || ws->rank != r || ws->device != wss[0]->device)
            return fail(GPUK_ERR_INVALID_ARGUMENT, "workspace %d does not belong to this emulated group", r);
        CallArgs a = {allreduce_in[r], residual_in, rms_gamma, fused ? residual_out[r] : nullptr,
                      fused ? norm_out[r] : nullptr, (fused && scale_out) ? scale_out[r] : nullptr,
                      numel, hidden, dtype, eps, quant_type};
        ArShape s;
        int rc = build_ar_call(ws, a, force_mode, true, &host_params[r], &s);
        ws->ready = nullptr;      // ready words apply to one call
        if (rc) return rc;
        if (r == 0) shape = s;
        else if (s.grid != shape.grid || s.threads != shape.threads || s.vpt != shape.vpt || s.two_shot != shape.two_shot ||
                 s.sym != shape.sym || s.ws != shape.ws)
            return fail(GPUK_ERR_INVALID_ARGUMENT, "ranks disagree on the launch shape");
    }
    gpuk_ws *w0 = wss[0];
    GPUK_CUDA(cudaSetDevice(w0->device));
    if (!w0->emul_params) GPUK_CUDA(cudaMalloc(&w0->emul_params, sizeof(ArParams) * kMaxRanks));
    cudaStream_t s = static_cast<cudaStream_t>(stream);
    GPUK_CUDA(cudaMemcpyAsync(w0->emul_params, host_params, sizeof(ArParams) * world_size, cudaMemcpyHostToDevice, s));
    GPUK_CUDA(cudaStreamSynchronize(s));   // host_params lives on this stack frame
    return by_dtype(dtype, [&](auto *t) {
        using T = std::remove_pointer_t<decltype(t)>;
        cudaError_t e = launch_ar_emulated<T>(w0->emul_params, shape, s);
        if (e != cudaSuccess) return fail(GPUK_ERR_CUDA, "cooperative launch failed: %s", cudaGetErrorString(e));
        return static_cast<int>(GPUK_OK);
    });
}

}  // extern "C"

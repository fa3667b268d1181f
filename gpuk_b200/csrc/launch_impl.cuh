// Definitions behind launch.cuh; included only by the per-type translation units.
#pragma once

#include <mutex>

#include "launch.cuh"

namespace gpuk {

template <typename T, int VPT>
static const void *norm_quant_fn() { return reinterpret_cast<const void *>(&fused_norm_quant_kernel<T, VPT>); }

template <typename T, int NR, int VPT, bool TWO_SHOT, bool FUSED>
static const void *ar_fn(bool emulated) {
    return emulated ? reinterpret_cast<const void *>(&ar_emulated_kernel<T, NR, VPT, TWO_SHOT, FUSED>)
                    : reinterpret_cast<const void *>(&ar_kernel<T, NR, VPT, TWO_SHOT, FUSED>);
}

template <typename T, int NR, int VPT>
static const void *ar_sym_fn(const ArShape &s, bool emulated) {
    if (!s.fused) return nullptr;   // the plain all-reduce uses the push exchange
    if (emulated) return s.sym == 1 ? reinterpret_cast<const void *>(&ar_sym_emulated_kernel<T, NR, VPT>) : nullptr;
    return s.sym == 2 ? reinterpret_cast<const void *>(&ar_sym_kernel<T, NR, VPT, true>)
                      : reinterpret_cast<const void *>(&ar_sym_kernel<T, NR, VPT, false>);
}

template <typename T, int NR, int VPT, bool FUSED>
static const void *ar_ws_fn(bool emulated) {
    return emulated ? reinterpret_cast<const void *>(&ar_ws_emulated_kernel<T, NR, VPT, FUSED>)
                    : reinterpret_cast<const void *>(&ar_ws_kernel<T, NR, VPT, FUSED>);
}

template <typename T, int NR, int VPT>
static const void *ar_fn_modes(const ArShape &s, bool emulated) {
    if (s.sym) return ar_sym_fn<T, NR, VPT>(s, emulated);
    if (s.ws == 2) {   // two ranks, one hop, fused operator
        if constexpr (NR == 2) {
            if (s.fused) return emulated ? reinterpret_cast<const void *>(&ar_ws1_emulated_kernel<T, VPT>)
                                         : reinterpret_cast<const void *>(&ar_ws1_kernel<T, VPT>);
        }
        return nullptr;
    }
    if (s.ws) {
        if (s.fused) return ar_ws_fn<T, NR, VPT, true>(emulated);
        if constexpr (VPT == 2) return ar_ws_fn<T, NR, VPT, false>(emulated);   // the plain all-reduce views rows of 1024 vectors
        return nullptr;
    }
    if (s.fused) return s.two_shot ? ar_fn<T, NR, VPT, true, true>(emulated) : ar_fn<T, NR, VPT, false, true>(emulated);
    if constexpr (VPT == 4) {   // the plain all-reduce is only built for the 4-vector tile
        return s.two_shot ? ar_fn<T, NR, VPT, true, false>(emulated) : ar_fn<T, NR, VPT, false, false>(emulated);
    }
    return nullptr;
}

template <typename T, int NR>
static const void *ar_fn_vpt(const ArShape &s, bool emulated) {
    switch (s.vpt) {
    case 1: return ar_fn_modes<T, NR, 1>(s, emulated);
    case 2: return ar_fn_modes<T, NR, 2>(s, emulated);
    case 4: return ar_fn_modes<T, NR, 4>(s, emulated);
    case 8: return ar_fn_modes<T, NR, 8>(s, emulated);
    default: return nullptr;
    }
}

template <typename T>
static const void *ar_fn_any(const ArShape &s, bool emulated) {
    switch (s.world) {
    case 2: return ar_fn_vpt<T, 2>(s, emulated);
    case 4: return ar_fn_vpt<T, 4>(s, emulated);
    case 8: return ar_fn_vpt<T, 8>(s, emulated);
    default: return nullptr;
    }
}

template <typename T>
cudaError_t launch_norm_quant(const NormQuantParams &p, int vpt, int threads, int grid, cudaStream_t stream) {
    const void *fn = nullptr;
    switch (vpt) {
    case 1: fn = norm_quant_fn<T, 1>(); break;
    case 2: fn = norm_quant_fn<T, 2>(); break;
    case 4: fn = norm_quant_fn<T, 4>(); break;
    case 8: fn = norm_quant_fn<T, 8>(); break;
    default: return cudaErrorInvalidValue;
    }
    NormQuantParams q = p;
    q.full = p.ep.row_vecs == vpt * threads ? 1 : 0;
    void *args[] = {&q};
    return launch_kernel(fn, grid, threads, 1, false, args, stream);
}

template <typename T, int VPT>
static cudaError_t launch_staged_one(const NormQuantParams &p0, int threads, int stages, int sm_count, int ctas_per_sm, cudaStream_t stream) {
    const void *fn = reinterpret_cast<const void *>(&fused_norm_quant_staged_kernel<T, VPT>);
    if (threads > tile_max_threads<VPT>()) return cudaErrorInvalidConfiguration;
    NormQuantParams p = p0;
    const size_t stage_bytes = static_cast<size_t>(2) * p.ep.row_vecs * 16;
    if (stages > kMaxStages) stages = kMaxStages;
    while (stages > 1 && stages * stage_bytes > 200 * 1024) --stages;
    const size_t smem = stages * stage_bytes;
    if (stages < 1 || smem > 200 * 1024) return cudaErrorInvalidConfiguration;
    p.stages = stages;
    p.full = p.ep.row_vecs == VPT * threads ? 1 : 0;
    // per device: opt in to the shared-memory size and look up how many CTAs fit an SM
    // (this entry point has no workspace to keep the cache in, so it is guarded for concurrent callers)
    static std::mutex cache_mutex;
    static int per_sm_by_device[64] = {};
    static size_t smem_by_device[64] = {};
    static int threads_by_device[64] = {};
    static size_t smem_max_by_device[64] = {};
    int device = 0;
    cudaError_t e = cudaGetDevice(&device);
    if (e != cudaSuccess) return e;
    if (device < 0 || device >= 64) return cudaErrorInvalidConfiguration;
    int per_sm;
    {
        std::lock_guard<std::mutex> lock(cache_mutex);
        if (per_sm_by_device[device] == 0 || smem_by_device[device] != smem || threads_by_device[device] != threads) {
            if (smem > smem_max_by_device[device]) {
                e = cudaFuncSetAttribute(fn, cudaFuncAttributeMaxDynamicSharedMemorySize, static_cast<int>(smem));
                if (e != cudaSuccess) return e;
                smem_max_by_device[device] = smem;
            }
            int n = 0;
            e = cudaOccupancyMaxActiveBlocksPerMultiprocessor(&n, fn, threads, smem);
            if (e != cudaSuccess) return e;
            if (n <= 0) return cudaErrorInvalidConfiguration;
            per_sm_by_device[device] = n;
            smem_by_device[device] = smem;
            threads_by_device[device] = threads;
        }
        per_sm = per_sm_by_device[device];
    }
    if (ctas_per_sm > 0 && ctas_per_sm < per_sm) per_sm = ctas_per_sm;
    const int64_t slots = static_cast<int64_t>(per_sm) * sm_count;
    // every CTA takes the same number of rows (the last ones one fewer): no ragged last wave
    const int64_t rounds = (p.rows + slots - 1) / slots;
    const int grid = static_cast<int>((p.rows + rounds - 1) / rounds);
    void *args[] = {&p};
    return launch_kernel(fn, grid, threads, 1, false, args, stream, smem);
}

template <typename T>
cudaError_t launch_norm_quant_staged(const NormQuantParams &p, int vpt, int threads, int stages, int sm_count, int ctas_per_sm,
                                     cudaStream_t stream) {
    if (threads < 64) return cudaErrorInvalidConfiguration;
    switch (vpt) {
    case 1: return launch_staged_one<T, 1>(p, threads, stages, sm_count, ctas_per_sm, stream);
    case 2: return launch_staged_one<T, 2>(p, threads, stages, sm_count, ctas_per_sm, stream);
    case 4: return launch_staged_one<T, 4>(p, threads, stages, sm_count, ctas_per_sm, stream);
    default: return cudaErrorInvalidConfiguration;
    }
}

template <typename T>
cudaError_t launch_ar(const ArParams &p, const ArShape &s, cudaStream_t stream) {
    const void *fn = ar_fn_any<T>(s, false);
    if (!fn) return cudaErrorInvalidValue;
    void *args[] = {const_cast<ArParams *>(&p)};
    return launch_kernel(fn, s.grid, s.threads, s.cluster, false, args, stream);
}

template <typename T>
cudaError_t launch_ar_emulated(const ArParams *params_by_rank, const ArShape &s, cudaStream_t stream) {
    const void *fn = ar_fn_any<T>(s, true);
    if (!fn) return cudaErrorInvalidValue;
    int nb = s.grid;
    void *args[] = {&params_by_rank, &nb};
    return launch_kernel(fn, s.grid * s.world, s.threads, s.cluster, true, args, stream);
}

template <typename T>
cudaError_t ar_resident_ctas(const ArShape &s, bool emulated, int sm_count, int64_t *ctas) {
    const void *fn = ar_fn_any<T>(s, emulated);
    if (!fn) return cudaErrorInvalidValue;
    return resident_ctas(fn, s.threads, s.cluster, sm_count, ctas);
}

#define GPUK_INSTANTIATE_LAUNCHERS(T)                                                                          \
    template cudaError_t launch_norm_quant<T>(const NormQuantParams &, int, int, int, cudaStream_t);           \
    template cudaError_t launch_norm_quant_staged<T>(const NormQuantParams &, int, int, int, int, int, cudaStream_t); \
    template cudaError_t launch_ar<T>(const ArParams &, const ArShape &, cudaStream_t);                        \
    template cudaError_t launch_ar_emulated<T>(const ArParams *, const ArShape &, cudaStream_t);               \
    template cudaError_t ar_resident_ctas<T>(const ArShape &, bool, int, int64_t *);

}  // namespace gpuk

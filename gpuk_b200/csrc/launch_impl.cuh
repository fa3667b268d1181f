// Definitions behind launch.cuh; included only by the per-type translation units.
#pragma once

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
static const void *ar_fn_modes(const ArShape &s, bool emulated) {
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
    void *args[] = {const_cast<NormQuantParams *>(&p)};
    return cudaLaunchKernel(fn, dim3(grid), dim3(threads), args, 0, stream);
}

template <typename T>
cudaError_t launch_ar(const ArParams &p, const ArShape &s, cudaStream_t stream) {
    const void *fn = ar_fn_any<T>(s, false);
    if (!fn) return cudaErrorInvalidValue;
    void *args[] = {const_cast<ArParams *>(&p)};
    return cudaLaunchKernel(fn, dim3(s.grid), dim3(s.threads), args, 0, stream);
}

template <typename T>
cudaError_t launch_ar_emulated(const ArParams *params_by_rank, const ArShape &s, cudaStream_t stream) {
    const void *fn = ar_fn_any<T>(s, true);
    if (!fn) return cudaErrorInvalidValue;
    int nb = s.grid;
    void *args[] = {&params_by_rank, &nb};
    return cudaLaunchCooperativeKernel(fn, dim3(s.grid * s.world), dim3(s.threads), args, 0, stream);
}

template <typename T>
cudaError_t ar_blocks_per_sm(const ArShape &s, bool emulated, int *blocks_per_sm) {
    const void *fn = ar_fn_any<T>(s, emulated);
    if (!fn) return cudaErrorInvalidValue;
    return cudaOccupancyMaxActiveBlocksPerMultiprocessor(blocks_per_sm, fn, s.threads, 0);
}

#define GPUK_INSTANTIATE_LAUNCHERS(T)                                                                          \
    template cudaError_t launch_norm_quant<T>(const NormQuantParams &, int, int, int, cudaStream_t);           \
    template cudaError_t launch_ar<T>(const ArParams &, const ArShape &, cudaStream_t);                        \
    template cudaError_t launch_ar_emulated<T>(const ArParams *, const ArShape &, cudaStream_t);               \
    template cudaError_t ar_blocks_per_sm<T>(const ArShape &, bool, int *);

}  // namespace gpuk

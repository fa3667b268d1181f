// Host-side launchers: turn runtime (world size, tile, mode) into a kernel instantiation.
// The templates are instantiated once per element type in launch_bf16.cu / _f16.cu / _f32.cu
// so the three translation units compile in parallel.
#pragma once

#include "kernels.cuh"

namespace gpuk {

struct ArShape {
    int world;       // 2, 4 or 8
    int vpt;         // 1, 2, 4 or 8 (plain all-reduce: 4 only)
    bool two_shot;
    bool fused;
    int threads;
    int grid;        // CTAs per rank
};

template <typename T>
cudaError_t launch_norm_quant(const NormQuantParams &p, int vpt, int threads, int grid, cudaStream_t stream);

template <typename T>
cudaError_t launch_ar(const ArParams &p, const ArShape &s, cudaStream_t stream);

// params_by_rank is a device array of s.world entries; the launch is cooperative.
template <typename T>
cudaError_t launch_ar_emulated(const ArParams *params_by_rank, const ArShape &s, cudaStream_t stream);

// Resident CTAs per SM of the instantiation `s` selects (emulated = the one-GPU variant).
template <typename T>
cudaError_t ar_blocks_per_sm(const ArShape &s, bool emulated, int *blocks_per_sm);

// Records the text gpuk_last_error() returns on this thread and hands `code` back
// (defined next to gpuk_last_error).
int set_last_error(int code, const char *fmt, ...);

}  // namespace gpuk

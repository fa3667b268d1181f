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
    int grid;        // CTAs per rank (a multiple of `cluster`)
    int cluster;     // CTAs per thread-block cluster (1: launched without a cluster attribute)
    int ws;          // 1: the warp-specialised two-shot kernel (vpt: vectors per finishing thread, threads: all roles);
                     // 2: its two-rank one-hop variant (finishing and pushing warps only)
    int sym;         // 0: push exchange; 1: exchange through symmetric memory with peer loads;
                     // 2: the same with NVSwitch multicast (two_shot is true for 1 and 2)
};

// Launches `fn` (one parameter block behind args) with an optional cluster dimension; with
// `all_resident` the launch is cooperative, i.e. refused unless the whole grid fits the GPU.
// Other launches are programmatic dependent launches : the kernels wait
// for the preceding grid themselves (griddepcontrol.wait) before they touch memory, so their
// CTAs may be placed on the SMs while the tail of the preceding kernel is still running.
cudaError_t launch_kernel(const void *fn, int grid, int threads, int cluster, bool all_resident, void **args, cudaStream_t stream,
                          size_t dynamic_smem = 0);
// CTAs of `fn` that can be resident on the whole GPU at once, counting whole clusters only.
cudaError_t resident_ctas(const void *fn, int threads, int cluster, int sm_count, int64_t *ctas);

template <typename T>
cudaError_t launch_norm_quant(const NormQuantParams &p, int vpt, int threads, int grid, cudaStream_t stream);

// Staged variant (rows through shared memory by bulk copies) on persistent CTAs: as many as fit
// the GPU at once (at most `ctas_per_sm` per SM if that is positive), but no more than it takes
// to give every CTA the same number of rows.  Returns cudaErrorInvalidConfiguration when the tile
// is not built or a row does not fit the shared memory, so that the caller can use the plain kernel.
template <typename T>
cudaError_t launch_norm_quant_staged(const NormQuantParams &p, int vpt, int threads, int stages, int sm_count, int ctas_per_sm,
                                     cudaStream_t stream);

template <typename T>
cudaError_t launch_ar(const ArParams &p, const ArShape &s, cudaStream_t stream);

// params_by_rank is a device array of s.world entries; the launch is cooperative.
template <typename T>
cudaError_t launch_ar_emulated(const ArParams *params_by_rank, const ArShape &s, cudaStream_t stream);

// CTAs of the instantiation `s` selects that fit the GPU at once (emulated = the one-GPU variant).
template <typename T>
cudaError_t ar_resident_ctas(const ArShape &s, bool emulated, int sm_count, int64_t *ctas);

// Process-wide tuning of the FP8 linear layer (gpuk_set_tuning "fp8_frags_per_warp"): 16-row fragments per warp,
// 1 or 2; 0 = chosen from the shape.  Defined in fp8_linear.cu.
extern int fp8_frags_per_warp_tuning;

// Quantisation policy of an operator quant_type (include/gpuk_b200.h); false for an unknown one.
bool quant_from_type(int quant_type, Quant *q);

// Records the text gpuk_last_error() returns on this thread and hands `code` back
// (defined next to gpuk_last_error).
int set_last_error(int code, const char *fmt, ...);

}  // namespace gpuk

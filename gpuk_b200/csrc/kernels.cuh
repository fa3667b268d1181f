// The kernels of the tensor-parallel epilogue, written for sm_100a.
//
//   fused_norm_quant_kernel   one GPU, no communication: residual add + RMSNorm + FP8.
//   ar_kernel                 N GPUs: all-reduce of the per-rank partials fused with the same
//                             epilogue (or, with FUSED = false, a plain all-reduce), as a
//                             one-shot (latency) or two-shot (bandwidth) exchange.
//   ar_emulated_kernel        the same device code run for N ranks inside ONE cooperative
//                             launch on one GPU, so that the multi-rank logic can be checked
//                             where only one GPU is available.
//
// They replace src/impl/all_reduce_fusion_impl.h:40-98 (allreduce_inplace_kernel_2stage),
// :230-268 (allreduce_fusion_kernel_1stage) and :285-346 (allreduce_fusion_kernel_2stage).
//
// Exchange design (differs from the reference on purpose).  The reference pulls: peers read
// each other's input, which therefore has to be copied into an IPC-visible staging buffer
// first (src/ops/all_reduce_fusion.cpp:129-132) or registered ahead of time.  Here every
// transfer is a push: a rank reads its own input from wherever it lives and writes 16-byte
// vectors straight into its peers' staging memory, then raises a flag there.  Nothing but
// the workspace is ever mapped across processes, there is no staging copy, and NVLink only
// carries posted writes.
//
//   one-shot   rank r writes its whole row into slot r of every peer; each rank then sums
//              the N slots locally in rank order (so all ranks get identical bits) and runs
//              the epilogue.  One flag hop.  Slots are double-buffered by call parity.
//   two-shot   a row is cut into N column slices; rank r writes slice j of its row into slot
//              r of rank j (reduce-scatter by push), rank j sums its N slots in rank order,
//              rounds once and writes the reduced slice into every rank's gather area
//              (all-gather by push); each rank then runs the epilogue on whole rows.  CTA b
//              on every rank works on the same rows, so all synchronisation is between CTAs
//              of equal index (the structural idea of communicator.h:82-88), and a CTA
//              software-pipelines its chunks: push k+1, reduce k, epilogue k-1.
//
// Every loop that moves data issues a batch of independent 16-byte loads before the first
// dependent store, because a store to memory that may alias the source stops the compiler
// from hoisting later loads above it.
#pragma once

#include "epilogue.cuh"

namespace gpuk {

template <int VPT>
constexpr int tile_max_threads() { return VPT == 4 ? 256 : (VPT == 8 ? 512 : 1024); }
template <int VPT>
constexpr int tile_min_blocks() { return VPT == 4 ? 4 : 1; }

// ---------------------------------------------------------------------------------------
// one GPU: residual add + RMSNorm + FP8, no communication
// ---------------------------------------------------------------------------------------
struct NormQuantParams {
    const void *in;     // [rows, hidden] T
    int64_t rows;
    EpilogueArgs ep;
};

template <typename T, int VPT>
__global__ void __launch_bounds__(tile_max_threads<VPT>(), tile_min_blocks<VPT>())
    fused_norm_quant_kernel(const __grid_constant__ NormQuantParams p) {
    __shared__ EpilogueSmem sm;
    const float static_scale = p.ep.q.mode == kQuantStatic ? *p.ep.scale_out : 1.f;
    int parity = 0;
    for (int64_t row = blockIdx.x; row < p.rows; row += gridDim.x, parity ^= 1) {
        const uint4 *src = reinterpret_cast<const uint4 *>(p.in) + row * p.ep.row_vecs;
        uint4 x[VPT], res[VPT];
#pragma unroll
        for (int i = 0; i < VPT; ++i) {
            const int v = threadIdx.x + i * blockDim.x;
            x[i] = v < p.ep.row_vecs ? ld_stream(src + v) : make_uint4(0, 0, 0, 0);
        }
        load_residual<T, VPT>(p.ep, row, res);
        row_epilogue<T, VPT>(p.ep, row, x, res, sm, parity, static_scale);
    }
}

// ---------------------------------------------------------------------------------------
// N GPUs
// ---------------------------------------------------------------------------------------
struct ArParams {
    // tensor
    const void *in;        // local partial, viewed as `rows` rows of `row_vecs` 16-byte vectors
    void *out;             // plain all-reduce only: destination (may alias `in`)
    int64_t total_vecs;    // vectors in the tensor (the last row may be shorter)
    int rows;
    int row_vecs;
    int rows_per_chunk;    // rows a CTA handles between two flag exchanges
    EpilogueArgs ep;       // fused only
    // communication
    int rank;
    int vpr;               // vectors of a row owned by one rank = ceil(row_vecs / N)
    char *peer_data[kMaxRanks];        // every rank's staging base as mapped here ([rank] is local)
    uint32_t *peer_flags[kMaxRanks];   // every rank's flag array as mapped here
    LocalState *st;
    int64_t rs_slot_bytes;   // two-shot: stride between the N reduce-scatter slots
    int64_t ag_off;          // two-shot: offset of the gather area
    int64_t os_off;          // one-shot: offset of buffer 0
    int64_t os_slot_bytes;   // one-shot: stride between slots; a buffer is N slots
    uint32_t epoch_advance;  // how far this call moves the flag epoch
    int roles;               // two-shot: 1 = every CTA runs all three stages of its chunks,
                             // 3 = CTAs specialise (3*lane + {0: push, 1: reduce+gather, 2: epilogue})
};

// `with_self`: also raise / await this rank's own flag.  Needed when the data of a stage is
// produced and consumed by different CTAs of the same rank (specialised roles).
template <int NR>
__device__ __forceinline__ void signal_peers(const ArParams &p, int stage, int vb, uint32_t value, bool with_self = false) {
    __syncthreads();   // every thread's pushes precede the release below (cumulativity)
    const int t = threadIdx.x;
    if (t < NR && (with_self || t != p.rank)) st_release_sys(p.peer_flags[t] + flag_index(stage, vb, p.rank), value);
}

template <int NR>
__device__ __forceinline__ void wait_peers(const ArParams &p, int stage, int vb, uint32_t value, bool with_self = false) {
    const int t = threadIdx.x;
    if (t < NR && (with_self || t != p.rank))
        wait_flag(p.peer_flags[p.rank] + flag_index(stage, vb, t), value, p.st, p.rank, vb, stage, t);
    __syncthreads();   // the acquire above now orders every thread's reads of the pushed data
}

__device__ __forceinline__ int row_len(const ArParams &p, int row) {
    const int64_t left = p.total_vecs - static_cast<int64_t>(row) * p.row_vecs;
    return left < p.row_vecs ? static_cast<int>(left) : p.row_vecs;
}

template <typename T, int NR>
__device__ __forceinline__ uint4 sum_in_rank_order(const uint4 (&part)[NR]) {
    constexpr int KV = Elem<T>::kVec;
    float acc[KV];
    Elem<T>::unpack(part[0], acc);
#pragma unroll
    for (int s = 1; s < NR; ++s) {
        float f[KV];
        Elem<T>::unpack(part[s], f);
#pragma unroll
        for (int e = 0; e < KV; ++e) acc[e] += f[e];
    }
    return Elem<T>::pack(acc);
}

// ---- two-shot stages -------------------------------------------------------------------

// Stage 1: scatter the slices of rows [r0, r1) of my partial to their owners.
template <typename T, int NR>
__device__ __forceinline__ void push_slices(const ArParams &p, int r0, int r1) {
    constexpr int U = 4;
    const uint4 *in = reinterpret_cast<const uint4 *>(p.in);
    const int B = blockDim.x;
    for (int row = r0; row < r1; ++row) {
        const int len = row_len(p, row);
        const int64_t base = static_cast<int64_t>(row) * p.row_vecs;
        for (int v0 = threadIdx.x; v0 < len; v0 += U * B) {
            uint4 val[U];
            int owner[U];
#pragma unroll
            for (int u = 0; u < U; ++u) {
                const int v = v0 + u * B;
                owner[u] = v < len ? v / p.vpr : p.rank;     // my own slice is summed straight from `in`
                if (owner[u] != p.rank) val[u] = ld_stream(in + base + v);
            }
#pragma unroll
            for (int u = 0; u < U; ++u) {
                const int v = v0 + u * B;
                if (owner[u] != p.rank) {
                    char *slot = p.peer_data[owner[u]] + p.rank * p.rs_slot_bytes;
                    st_peer(reinterpret_cast<uint4 *>(slot) + static_cast<int64_t>(row) * p.vpr + (v - owner[u] * p.vpr), val[u]);
                }
            }
        }
    }
}

// Stage 2: sum my slice of rows [r0, r1) over all ranks in rank order, round once, and
// write the result into every rank's gather area.
template <typename T, int NR>
__device__ __forceinline__ void reduce_and_gather(const ArParams &p, int r0, int r1) {
    constexpr int IB = NR >= 8 ? 1 : (NR == 4 ? 2 : 4);   // items per batch: ~8 loads in flight per thread
    const uint4 *in = reinterpret_cast<const uint4 *>(p.in);
    const int items = (r1 - r0) * p.vpr;
    const int B = blockDim.x;
    for (int it0 = threadIdx.x; it0 < items; it0 += IB * B) {
        uint4 part[IB][NR];
        int64_t dst[IB];
#pragma unroll
        for (int b = 0; b < IB; ++b) {
            const int it = it0 + b * B;
            dst[b] = -1;
            if (it < items) {
                const int rr = it / p.vpr;
                const int vl = it - rr * p.vpr;
                const int row = r0 + rr;
                const int v = p.rank * p.vpr + vl;
                if (v < row_len(p, row)) {
                    dst[b] = static_cast<int64_t>(row) * p.row_vecs + v;
#pragma unroll
                    for (int s = 0; s < NR; ++s) {
                        if (s == p.rank) {
                            part[b][s] = ld_stream(in + dst[b]);
                        } else {
                            const char *slot = p.peer_data[p.rank] + s * p.rs_slot_bytes;
                            part[b][s] = ld_staging(reinterpret_cast<const uint4 *>(slot) + static_cast<int64_t>(row) * p.vpr + vl);
                        }
                    }
                }
            }
        }
#pragma unroll
        for (int b = 0; b < IB; ++b) {
            if (dst[b] >= 0) {
                const uint4 red = sum_in_rank_order<T, NR>(part[b]);
#pragma unroll
                for (int d = 0; d < NR; ++d) {
                    const int j = (p.rank + d) % NR;   // start with myself, then fan out: spreads the links
                    st_peer(reinterpret_cast<uint4 *>(p.peer_data[j] + p.ag_off) + dst[b], red);
                }
            }
        }
    }
}

// Stage 3: rows [r0, r1) are complete in my gather area.
template <typename T, int NR, int VPT, bool FUSED>
__device__ __forceinline__ void finish_rows(const ArParams &p, int r0, int r1, EpilogueSmem &sm, int &parity,
                                            float static_scale) {
    const uint4 *ag = reinterpret_cast<const uint4 *>(p.peer_data[p.rank] + p.ag_off);
    for (int row = r0; row < r1; ++row) {
        const int64_t base = static_cast<int64_t>(row) * p.row_vecs;
        if constexpr (FUSED) {
            uint4 x[VPT], res[VPT];
#pragma unroll
            for (int i = 0; i < VPT; ++i) {
                const int v = threadIdx.x + i * blockDim.x;
                x[i] = v < p.row_vecs ? ld_staging(ag + base + v) : make_uint4(0, 0, 0, 0);
            }
            load_residual<T, VPT>(p.ep, row, res);
            row_epilogue<T, VPT>(p.ep, row, x, res, sm, parity, static_scale);
            parity ^= 1;
        } else {
            constexpr int U = 4;
            const int len = row_len(p, row);
            const int B = blockDim.x;
            for (int v0 = threadIdx.x; v0 < len; v0 += U * B) {
                uint4 val[U];
#pragma unroll
                for (int u = 0; u < U; ++u)
                    if (v0 + u * B < len) val[u] = ld_staging(ag + base + v0 + u * B);
#pragma unroll
                for (int u = 0; u < U; ++u)
                    if (v0 + u * B < len) st_stream(reinterpret_cast<uint4 *>(p.out) + base + v0 + u * B, val[u]);
            }
        }
    }
}

// ---- the body: one CTA of one rank ------------------------------------------------------
template <typename T, int NR, int VPT, bool TWO_SHOT, bool FUSED>
__device__ __forceinline__ void ar_body(const ArParams &p, int vb, int nb, EpilogueSmem &sm) {
    LocalState *st = p.st;
    const uint32_t base = ld_volatile_u32(&st->epoch);
    float static_scale = 1.f;
    if constexpr (FUSED) {
        if (p.ep.q.mode == kQuantStatic) static_scale = *p.ep.scale_out;
    }
    int parity = 0;
    const int R = p.rows_per_chunk;
    const int nchunks = (p.rows + R - 1) / R;
    const int nk = vb < nchunks ? (nchunks - vb + nb - 1) / nb : 0;   // chunks of this CTA: vb, vb+nb, ...

    if (TWO_SHOT && p.roles == 3) {
        // Specialised roles: the three stages of a lane's chunks run in three CTAs that only meet
        // through flags, so pushes stream without ever waiting, reductions start as soon as a
        // chunk has landed, and the epilogue trails behind -- the stages of different chunks
        // overlap in time even when a lane owns only a few chunks.
        const int lanes = nb / 3, lane = vb / 3, role = vb - lane * 3;
        const int nl = lane < nchunks ? (nchunks - lane + lanes - 1) / lanes : 0;
        for (int k = 0; k < nl; ++k) {
            const int r0 = (lane + k * lanes) * R;
            const int r1 = r0 + R < p.rows ? r0 + R : p.rows;
            if (role == 0) {
                push_slices<T, NR>(p, r0, r1);
                signal_peers<NR>(p, 0, lane, base + k + 1);
            } else if (role == 1) {
                wait_peers<NR>(p, 0, lane, base + k + 1);
                reduce_and_gather<T, NR>(p, r0, r1);
                signal_peers<NR>(p, 1, lane, base + k + 1, true);
            } else {
                wait_peers<NR>(p, 1, lane, base + k + 1, true);
                finish_rows<T, NR, VPT, FUSED>(p, r0, r1, sm, parity, static_scale);
            }
        }
    } else if constexpr (TWO_SHOT) {
        auto r0_of = [&](int k) { return (vb + k * nb) * R; };
        auto r1_of = [&](int k) { const int r1 = (vb + k * nb) * R + R; return r1 < p.rows ? r1 : p.rows; };
        if (nk > 0) {
            push_slices<T, NR>(p, r0_of(0), r1_of(0));
            signal_peers<NR>(p, 0, vb, base + 1);
        }
        for (int k = 0; k < nk; ++k) {
            if (k + 1 < nk) {
                push_slices<T, NR>(p, r0_of(k + 1), r1_of(k + 1));
                signal_peers<NR>(p, 0, vb, base + k + 2);
            }
            wait_peers<NR>(p, 0, vb, base + k + 1);
            reduce_and_gather<T, NR>(p, r0_of(k), r1_of(k));
            signal_peers<NR>(p, 1, vb, base + k + 1);
            if (k > 0) {
                wait_peers<NR>(p, 1, vb, base + k);
                finish_rows<T, NR, VPT, FUSED>(p, r0_of(k - 1), r1_of(k - 1), sm, parity, static_scale);
            }
        }
        if (nk > 0) {
            wait_peers<NR>(p, 1, vb, base + nk);
            finish_rows<T, NR, VPT, FUSED>(p, r0_of(nk - 1), r1_of(nk - 1), sm, parity, static_scale);
        }
    } else {
        // one-shot: one row per step, no pipelining (the regime is a handful of rows per CTA)
        const uint32_t buf = ld_volatile_u32(&st->os_seq) & 1u;
        const int64_t buf_off = p.os_off + static_cast<int64_t>(buf) * NR * p.os_slot_bytes;
        const uint4 *in = reinterpret_cast<const uint4 *>(p.in);
        for (int k = 0; k < nk; ++k) {
            const int row = vb + k * nb;   // rows_per_chunk is 1 on this path
            const int len = row_len(p, row);
            const int64_t rbase = static_cast<int64_t>(row) * p.row_vecs;
            uint4 x[VPT], res[VPT];
#pragma unroll
            for (int i = 0; i < VPT; ++i) {
                const int v = threadIdx.x + i * blockDim.x;
                x[i] = v < len ? ld_stream(in + rbase + v) : make_uint4(0, 0, 0, 0);
            }
#pragma unroll
            for (int i = 0; i < VPT; ++i) {
                const int v = threadIdx.x + i * blockDim.x;
                if (v < len) {
#pragma unroll
                    for (int d = 1; d < NR; ++d) {
                        const int j = (p.rank + d) % NR;
                        st_peer(reinterpret_cast<uint4 *>(p.peer_data[j] + buf_off + p.rank * p.os_slot_bytes) + rbase + v, x[i]);
                    }
                }
            }
            signal_peers<NR>(p, 0, vb, base + k + 1);
            if constexpr (FUSED) load_residual<T, VPT>(p.ep, row, res);   // in flight while the peers' pushes arrive
            wait_peers<NR>(p, 0, vb, base + k + 1);
#pragma unroll
            for (int i = 0; i < VPT; ++i) {
                const int v = threadIdx.x + i * blockDim.x;
                if (v < len) {
                    uint4 part[NR];
#pragma unroll
                    for (int s = 0; s < NR; ++s) {
                        part[s] = s == p.rank
                                      ? x[i]
                                      : ld_staging(reinterpret_cast<const uint4 *>(p.peer_data[p.rank] + buf_off +
                                                                                   s * p.os_slot_bytes) + rbase + v);
                    }
                    x[i] = sum_in_rank_order<T, NR>(part);
                }
            }
            if constexpr (FUSED) {
                row_epilogue<T, VPT>(p.ep, row, x, res, sm, parity, static_scale);
                parity ^= 1;
            } else {
#pragma unroll
                for (int i = 0; i < VPT; ++i) {
                    const int v = threadIdx.x + i * blockDim.x;
                    if (v < len) st_stream(reinterpret_cast<uint4 *>(p.out) + rbase + v, x[i]);
                }
            }
        }
    }

    // the last CTA of this rank to finish moves the epoch on for the next call
    __syncthreads();
    if (threadIdx.x == 0) {
        __threadfence();
        const uint32_t done = atomicAdd(&st->ticket, 1u);
        if (done == static_cast<uint32_t>(nb) - 1u) {
            st->ticket = 0;
            st->epoch = base + p.epoch_advance;
            if constexpr (!TWO_SHOT) st->os_seq = st->os_seq + 1u;
            __threadfence();
        }
    }
}

template <typename T, int NR, int VPT, bool TWO_SHOT, bool FUSED>
__global__ void __launch_bounds__(tile_max_threads<VPT>(), tile_min_blocks<VPT>())
    ar_kernel(const __grid_constant__ ArParams p) {
    __shared__ EpilogueSmem sm;
    ar_body<T, NR, VPT, TWO_SHOT, FUSED>(p, blockIdx.x, gridDim.x, sm);
}

// N ranks in one cooperative launch on one GPU: block b plays CTA (b % nb) of rank (b / nb).
// All blocks are co-resident (cooperative launch), so the flag waits between "ranks" are safe.
template <typename T, int NR, int VPT, bool TWO_SHOT, bool FUSED>
__global__ void __launch_bounds__(tile_max_threads<VPT>(), tile_min_blocks<VPT>())
    ar_emulated_kernel(const ArParams *params_by_rank, int nb) {
    __shared__ EpilogueSmem sm;
    __shared__ ArParams p;
    const int rank = blockIdx.x / nb;
    for (int i = threadIdx.x; i < static_cast<int>(sizeof(ArParams) / 4); i += blockDim.x)
        reinterpret_cast<uint32_t *>(&p)[i] = reinterpret_cast<const uint32_t *>(params_by_rank + rank)[i];
    __syncthreads();
    ar_body<T, NR, VPT, TWO_SHOT, FUSED>(p, blockIdx.x % nb, nb, sm);
}

}  // namespace gpuk

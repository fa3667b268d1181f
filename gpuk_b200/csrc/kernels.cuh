// The kernels of the tensor-parallel epilogue, written for sm_100a.
//
//   fused_norm_quant_kernel   one GPU, no communication: residual add + RMSNorm + FP8.
//   fused_norm_quant_staged_kernel   the same for many rows, rows staged through shared memory
//                             by bulk copies.
//   ar_kernel                 N GPUs: all-reduce of the per-rank partials fused with the same
//                             epilogue (or, with FUSED = false, a plain all-reduce), as a
//                             one-shot (latency) or two-shot (bandwidth) exchange.
//   ar_sym_kernel             N GPUs, bandwidth regime: the exchange through symmetric memory,
//                             reduced inside the NVSwitch (multimem) where a multicast mapping
//                             exists; fused with the same epilogue.
//   ar_emulated_kernel        the same device code run for N ranks inside ONE cooperative
//                             launch on one GPU, so that the multi-rank logic can be checked
//                             where only one GPU is available.
//
// They replace src/impl/all_reduce_fusion_impl.h:40-98 (allreduce_inplace_kernel_2stage),
// :230-268 (allreduce_fusion_kernel_1stage) and :285-346 (allreduce_fusion_kernel_2stage).
//
// Exchange design (differs from the reference on purpose).  The reference pulls: peers read
// each other's input, which therefore has to be copied into an IPC-visible staging buffer
// first (src/ops/all_reduce_fusion.cpp:129-132) or registered ahead of time, and every stage
// is fenced by a counter barrier (src/common/communicator.h:79-113).  Here every transfer is
// a push of self-announcing data (see common.cuh): a rank reads its own input from wherever
// it lives and writes 16-byte vectors straight into its peers' staging memory; the receiver
// polls exactly the vectors it needs, consumes them, and puts the location back to rest.
// There are no flags, no fences and no barriers between GPUs, nothing but the workspace is
// ever mapped across processes, there is no staging copy, and NVLink only carries posted
// writes of payload.
//
//   one-shot   rank r writes its whole row into slot r of every peer; each rank then sums
//              the N slots locally in rank order (so all ranks get identical bits) and runs
//              the epilogue.
//   two-shot   a row is cut into N column slices; rank r writes slice j of its row into slot
//              r of rank j (reduce-scatter by push), rank j sums its N slots in rank order,
//              rounds once and writes the reduced slice into every rank's gather area
//              (all-gather by push); each rank then runs the epilogue on whole rows.  CTA b
//              on every rank works on the same rows (the structural idea of
//              communicator.h:82-88), and a CTA staggers its chunks -- scatter k+1, reduce k,
//              epilogue k-1 -- with the loads of the three roles in flight together.
//
// Staging is double-buffered by call parity (a device-side counter that the kernel advances
// itself, so a replayed CUDA graph stays in step): a rank can start call c+2 only after every peer has pushed its call c+1
// data, i.e. after every peer's call c kernel -- including its consume-and-reset of buffer
// c % 2 -- has completed.
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
constexpr int tile_min_blocks() { return VPT == 4 ? 4 : 1; }      // one-GPU kernel: 64 registers
template <int VPT>
constexpr int ar_min_blocks() { return VPT == 4 ? 3 : 1; }        // exchange kernels hold N vectors per item
// The two-shot exchange always runs on the bandwidth tile (at most 256 threads, 512 for the
// longest rows) and keeps the loads of three pipeline roles in registers: 128 registers.
template <int VPT, bool TWO_SHOT>
constexpr int ar_max_threads() { return TWO_SHOT ? (VPT == 8 ? 512 : 256) : tile_max_threads<VPT>(); }
template <int VPT, bool TWO_SHOT>
constexpr int ar_resident_blocks() { return TWO_SHOT ? (VPT == 8 ? 1 : 2) : ar_min_blocks<VPT>(); }

// ---------------------------------------------------------------------------------------
// one GPU: residual add + RMSNorm + FP8, no communication
// ---------------------------------------------------------------------------------------
struct NormQuantParams {
    const void *in;     // [rows, hidden] T
    int64_t rows;
    int stages;         // staged kernel: depth of the shared-memory ring (2 .. kMaxStages)
    int full;           // 1: a row is exactly VPT * blockDim vectors (the launcher sets it): no bounds checks
    EpilogueArgs ep;
};
constexpr int kMaxStages = 8;

template <typename T, int VPT, bool FULL>
__device__ __forceinline__ void norm_quant_rows(const NormQuantParams &p, EpilogueSmem &sm) {
    const float static_scale = p.ep.q.mode == kQuantStatic ? *p.ep.scale_out : 1.f;
    int parity = 0;
    for (int64_t row = blockIdx.x; row < p.rows; row += gridDim.x, parity ^= 1) {
        const uint4 *src = reinterpret_cast<const uint4 *>(p.in) + row * p.ep.row_vecs;
        uint4 x[VPT], res[VPT];
#pragma unroll
        for (int i = 0; i < VPT; ++i) {
            const int v = threadIdx.x + i * blockDim.x;
            x[i] = (FULL || v < p.ep.row_vecs) ? ld_stream(src + v) : make_uint4(0, 0, 0, 0);
        }
        const RowSeg seg = whole_row(p.ep.row_vecs);
        load_residual<T, VPT, FULL>(p.ep, seg, row, whole_cta(), res);
        row_epilogue<T, VPT, FULL>(p.ep, seg, row, whole_cta(), x, res, sm, parity, static_scale);
    }
}

template <typename T, int VPT>
__global__ void __launch_bounds__(tile_max_threads<VPT>(), tile_min_blocks<VPT>())
    fused_norm_quant_kernel(const __grid_constant__ NormQuantParams p) {
    __shared__ EpilogueSmem sm;
    grid_dependency_sync();
    if (p.full) norm_quant_rows<T, VPT, true>(p, sm);
    else norm_quant_rows<T, VPT, false>(p, sm);
}

// The same operation on persistent CTAs: each takes rows blockIdx.x, + gridDim.x, ... and fetches
// every row (input and residual, contiguous in global memory) into a ring of `stages`
// shared-memory stages with two bulk copies that one thread issues.  A stage is refilled with
// the row `stages` ahead as soon as every thread has taken its vectors out of it, so the loads of
// the next rows are in flight during both block reductions of the current one and the GPU's
// memory system sees reads, arithmetic and writes of different rows at the same time.
// Dynamic shared memory: stages * 2 * row_vecs * 16 bytes.  Needs at least two warps per CTA
// (the refill relies on the block barrier inside the first reduction).
template <int VPT>
constexpr int staged_min_blocks() { return VPT == 4 ? 3 : 1; }

struct StagedSmem {
    EpilogueSmem ep;
    alignas(8) uint64_t full[kMaxStages];
};

template <typename T, int VPT, bool FULL>
__device__ __forceinline__ void norm_quant_staged_rows(const NormQuantParams &p, unsigned char *stage_mem, StagedSmem &sm) {
    uint64_t *full = sm.full;
    const int stages = p.stages;
    const uint32_t row_bytes = static_cast<uint32_t>(p.ep.row_vecs) * 16u;
    const int64_t nk = blockIdx.x < p.rows ? (p.rows - blockIdx.x + gridDim.x - 1) / gridDim.x : 0;
    auto issue = [&](int64_t k, int s) {
        const int64_t row = blockIdx.x + k * gridDim.x;
        unsigned char *dst = stage_mem + static_cast<size_t>(s) * 2 * row_bytes;
        mbar_expect_bytes(&full[s], 2 * row_bytes);
        bulk_load(dst, static_cast<const unsigned char *>(p.in) + row * row_bytes, row_bytes, &full[s]);
        bulk_load(dst + row_bytes, static_cast<const unsigned char *>(p.ep.residual) + row * row_bytes, row_bytes, &full[s]);
    };
    if (threadIdx.x == 0) {
        for (int s = 0; s < stages; ++s) mbar_init(&full[s], 1);
        mbar_init_fence();
        for (int64_t k = 0; k < stages && k < nk; ++k) issue(k, static_cast<int>(k));
    }
    __syncthreads();
    const float static_scale = p.ep.q.mode == kQuantStatic ? *p.ep.scale_out : 1.f;
    const RowSeg seg = whole_row(p.ep.row_vecs);
    int s = 0;
    uint32_t phase = 0;
    for (int64_t k = 0; k < nk; ++k) {
        mbar_wait(&full[s], phase);
        const uint4 *sx = reinterpret_cast<const uint4 *>(stage_mem + static_cast<size_t>(s) * 2 * row_bytes);
        const uint4 *sr = sx + p.ep.row_vecs;
        uint4 x[VPT], res[VPT];
#pragma unroll
        for (int i = 0; i < VPT; ++i) {
            const int v = threadIdx.x + i * blockDim.x;
            x[i] = (FULL || v < p.ep.row_vecs) ? sx[v] : make_uint4(0, 0, 0, 0);
            res[i] = (FULL || v < p.ep.row_vecs) ? sr[v] : make_uint4(0, 0, 0, 0);
        }
        row_epilogue<T, VPT, FULL>(p.ep, seg, blockIdx.x + k * gridDim.x, whole_cta(), x, res, sm.ep, static_cast<int>(k & 1), static_scale,
                                   [&] { if (threadIdx.x == 0 && k + stages < nk) issue(k + stages, s); });
        if (++s == stages) { s = 0; phase ^= 1u; }
    }
}

template <typename T, int VPT>
__global__ void __launch_bounds__(tile_max_threads<VPT>(), staged_min_blocks<VPT>())
    fused_norm_quant_staged_kernel(const __grid_constant__ NormQuantParams p) {
    extern __shared__ __align__(128) unsigned char stage_mem[];
    __shared__ StagedSmem sm;
    grid_dependency_sync();
    if (p.full) norm_quant_staged_rows<T, VPT, true>(p, stage_mem, sm);
    else norm_quant_staged_rows<T, VPT, false>(p, stage_mem, sm);
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
    int rows_per_chunk;    // rows a CTA moves through one stage before it turns to the next stage
    int seg_vecs;          // vectors of a row held by one CTA of the cluster that owns the row (all of them without a cluster)
    int cluster;           // CTAs per thread-block cluster the host planned (seg_vecs was sized for it); checked at entry
    int tf, tr, ts;        // warp-specialised two-shot: threads that finish rows / reduce slices / scatter (multiples of 32)
    int scatter_lead;      // ... rows the scattering warps may run ahead of the finishing warps of their CTA (0: unbounded)
    int full;              // ... 1: a row is exactly VPT * tf vectors, no bounds checks in the finishing warps
    int one_hop;           // ... two ranks only, 1: whole rows go straight to the peer's gather area and the finishing warps add
                           //     their own row: one NVLink hop instead of two for the same bytes on the wire
    int lead_push;         // two-shot: chunks by which the scatter runs ahead of the reduction (>= 1)
    int lead_reduce;       // two-shot: chunks by which the reduction runs ahead of the epilogue (>= 1)
    EpilogueArgs ep;       // fused only
    // communication
    int rank;
    int vpr;               // vectors of a row owned by one rank = ceil(row_vecs / N)
    char *peer_data[kMaxRanks];   // every rank's staging base as mapped here ([rank] is local)
    LocalState *st;
    int64_t rs_slot_bytes;   // two-shot: stride between the N scatter slots of a buffer
    int64_t ag_off;          // two-shot: offset of the gather area inside a buffer
    // warp-specialised two-shot: every rank's gather area as mapped here, the distance between its two
    // call-parity copies, and -- where the gather areas lie in symmetric memory behind one NVSwitch multicast
    // address -- that address: one store then lands in every rank's gather area (nullptr: one store per rank)
    char *ag_base[kMaxRanks];
    int64_t ag_stride;
    char *ag_mc;
    // warp-specialised two-shot: the input may still be in the making.  Word row / ready_rows of `ready` reaches
    // ready_value once those rows of `in` are complete; the scattering and reducing warps wait for it before they
    // read a row (nullptr: the whole input is there when the kernel starts).
    const uint32_t *ready;
    int ready_rows;
    uint32_t ready_value;
    int64_t ts_stride;       // two-shot: bytes between buffer 0 and buffer 1
    int64_t os_off;          // one-shot: offset of buffer 0
    int64_t os_slot_bytes;   // one-shot: stride between slots; a buffer is N slots
    // exchange through symmetric memory (ar_sym_kernel): the same layout in every rank's buffer
    char *sym[kMaxRanks];    // every rank's symmetric buffer as mapped here ([rank] is local)
    char *sym_mc;            // NVSwitch multicast mapping of those buffers (nullptr: none)
    int64_t sym_in_off;      // copy of the rank's input, laid out like the input
    int64_t sym_out_off;     // the reduced tensor, laid out like the input
    int64_t sym_flag_off;    // uint64 flags[2][kMaxBlocks][kMaxRanks], written by the rank of the last index
};

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

// ---- one pipeline step with all of its loads in flight together ----------------------------
// Scatter of row `row_a`, reduction of this rank's slice of row `row_b` and finish of row
// `row_c` (a negative row: nothing to do in that role).  The three roles belong to three
// different chunks of the CTA's pipeline and do not depend on one another, so their loads --
// the row of the input, the N slot vectors, the gathered row and its residual -- are issued back
// to back before anything is consumed: a step exposes one memory round trip instead of three.
template <typename T, int NR, int VPT, bool FUSED>
__device__ __forceinline__ void two_shot_step(const ArParams &p, int64_t ts, int row_a, int row_b, int row_c,
                                              int cl_rank, int cl_size, EpilogueSmem &sm, int &parity, float static_scale) {
    constexpr int IBB = (VPT + NR - 1) / NR;     // slice vectors per thread: a CTA's share of vpr <= VPT * blockDim / NR
    const uint4 *in = reinterpret_cast<const uint4 *>(p.in);
    char *mine = p.peer_data[p.rank] + ts;
    uint4 *ag = reinterpret_cast<uint4 *>(mine + p.ag_off);
    const int B = blockDim.x;
    // this CTA's segment of a row (the whole row unless a cluster shares it) and its share of the slice
    const int v0 = cl_rank * p.seg_vecs;
    const int sub = (p.vpr + cl_size - 1) / cl_size, vl0 = cl_rank * sub;
    const int vl1 = vl0 + sub < p.vpr ? vl0 + sub : p.vpr;
    auto seg_end = [&](int len) { return v0 + p.seg_vecs < len ? v0 + p.seg_vecs : len; };
    const int end_a = row_a >= 0 ? seg_end(row_len(p, row_a)) : 0;
    const int len_b = row_b >= 0 ? row_len(p, row_b) : 0;
    const int end_c = row_c >= 0 ? seg_end(row_len(p, row_c)) : 0;
    const int64_t base_a = static_cast<int64_t>(row_a) * p.row_vecs;
    const int64_t base_b = static_cast<int64_t>(row_b) * p.row_vecs;
    const int64_t base_c = static_cast<int64_t>(row_c) * p.row_vecs;
    const int64_t slot_b = static_cast<int64_t>(row_b) * p.vpr;

    // ---- issue: scatter
    uint4 a[VPT];
    int owner[VPT];
#pragma unroll
    for (int i = 0; i < VPT; ++i) {
        const int v = v0 + threadIdx.x + i * B;
        owner[i] = v < end_a ? v / p.vpr : p.rank;     // my own slice is summed straight from `in`
        if (owner[i] != p.rank) a[i] = ld_stream(in + base_a + v);
    }
    // ---- issue: reduction
    uint4 part[IBB][NR];
    bool have[IBB];
#pragma unroll
    for (int b = 0; b < IBB; ++b) {
        const int vl = vl0 + threadIdx.x + b * B;
        have[b] = vl < vl1 && p.rank * p.vpr + vl < len_b;
        if (have[b]) {
#pragma unroll
            for (int s2 = 0; s2 < NR; ++s2)
                part[b][s2] = s2 == p.rank ? ld_stream(in + base_b + p.rank * p.vpr + vl)
                                           : ld_poll(reinterpret_cast<const uint4 *>(mine + s2 * p.rs_slot_bytes) + slot_b + vl);
        }
    }
    // ---- issue: finish
    uint4 x[VPT], res[VPT];
#pragma unroll
    for (int i = 0; i < VPT; ++i) {
        const int v = v0 + threadIdx.x + i * B;
        x[i] = v < end_c ? ld_poll(ag + base_c + v) : make_uint4(0, 0, 0, 0);
    }
    const RowSeg seg = RowSeg{v0, end_c, cl_rank, cl_size};
    if constexpr (FUSED) {
        if (row_c >= 0) load_residual<T, VPT>(p.ep, seg, row_c, whole_cta(), res);
    }

    // ---- consume: scatter
#pragma unroll
    for (int i = 0; i < VPT; ++i) {
        const int v = v0 + threadIdx.x + i * B;
        if (owner[i] != p.rank) {
            char *slot = p.peer_data[owner[i]] + ts + p.rank * p.rs_slot_bytes;
            st_peer(reinterpret_cast<uint4 *>(slot) + static_cast<int64_t>(row_a) * p.vpr + (v - owner[i] * p.vpr), payload<T>(a[i]));
        }
    }
    // ---- consume: reduction, then gather by push
#pragma unroll
    for (int b = 0; b < IBB; ++b) {
        if (have[b]) {
            const int vl = vl0 + threadIdx.x + b * B;
#pragma unroll
            for (int s2 = 0; s2 < NR; ++s2) {
                if (s2 != p.rank) {
                    uint4 *addr = reinterpret_cast<uint4 *>(mine + s2 * p.rs_slot_bytes) + slot_b + vl;
                    part[b][s2] = wait_landed(addr, part[b][s2], p.st, p.rank, kStageScatter, s2);
                    st_empty(addr);
                }
            }
            const uint4 red = payload<T>(sum_in_rank_order<T, NR>(part[b]));
            const int64_t dst = base_b + p.rank * p.vpr + vl;
#pragma unroll
            for (int d = 0; d < NR; ++d) {
                const int j = (p.rank + d) % NR;   // start with myself, then fan out: spreads the links
                st_peer(reinterpret_cast<uint4 *>(p.peer_data[j] + ts + p.ag_off) + dst, red);
            }
        }
    }
    // ---- consume: finish
    if (row_c >= 0) {
#pragma unroll
        for (int i = 0; i < VPT; ++i) {
            const int v = v0 + threadIdx.x + i * B;
            if (v < end_c) {
                x[i] = wait_landed(ag + base_c + v, x[i], p.st, p.rank, kStageGather, v / p.vpr);
                st_empty(ag + base_c + v);
            }
        }
        if constexpr (FUSED) {
            row_epilogue<T, VPT>(p.ep, seg, row_c, whole_cta(), x, res, sm, parity, static_scale);
            parity ^= 1;
        } else {
#pragma unroll
            for (int i = 0; i < VPT; ++i) {
                const int v = v0 + threadIdx.x + i * B;
                if (v < end_c) st_stream(reinterpret_cast<uint4 *>(p.out) + base_c + v, x[i]);
            }
        }
    }
}

// ---- the body: one CTA of one rank ------------------------------------------------------

// Takes this CTA's ticket of the call and learns the call's number from the same atomic:
// LocalState::seq holds the number of completed exchanges in its upper 48 bits (the low bit
// of that number selects the staging buffer of this call) and the tickets taken so far by
// CTAs of the running call in its lower 16 bits.  The CTA that takes the last ticket clears
// the tickets and advances the number; every CTA of the call has read it by then, so the new
// value is first seen by the next launch.  One thread does it and shares the number through
// `sm.seq`; the caller passes a block barrier before reading it.
__device__ __forceinline__ void begin_call(LocalState *st, int nb, EpilogueSmem &sm) {
    if (threadIdx.x == 0) {
        const unsigned long long old = atomicAdd(&st->seq, 1ull);
        sm.seq = old >> 16;
        if ((old & 0xffffull) == static_cast<unsigned long long>(nb) - 1ull) atomicAdd(&st->seq, 0x10000ull - static_cast<unsigned long long>(nb));
    }
}

template <typename T, int NR, int VPT, bool TWO_SHOT, bool FUSED>
__device__ __forceinline__ void ar_body(const ArParams &p, int vb, int nb, EpilogueSmem &sm) {
    LocalState *st = p.st;
    float static_scale = 1.f;
    if constexpr (FUSED) {
        if (p.ep.q.mode == kQuantStatic) static_scale = *p.ep.scale_out;
    }
    int parity = 0;
    const int R = p.rows_per_chunk;
    const int nchunks = (p.rows + R - 1) / R;
    // The segments of a row were sized for the planned cluster.  In a launch whose cluster attribute
    // did not take effect a CTA would handle segment 0 only and leave the rest of every row unwritten:
    // report it instead, before any ticket is taken or byte is stored.
    if (cluster_size() != p.cluster) {
        if (threadIdx.x == 0) record_status(st, kStatusClusterMismatch, p.rank, vb, TWO_SHOT ? kStageScatter : kStageOneShot, p.rank, cluster_size());
        return;
    }

    if constexpr (TWO_SHOT) {
        begin_call(st, nb, sm);
        __syncthreads();
        const int64_t ts = static_cast<int64_t>(sm.seq & 1ull) * p.ts_stride;
        // Every CTA takes its chunks (vb, vb + nb, ...) through the three roles as a software
        // pipeline: in step s it scatters chunk s, reduces chunk s - lead_push and finishes chunk
        // s - lead_push - lead_reduce, row by row, so that traffic for later chunks is on the wire
        // while the epilogue of an earlier one runs.  Nothing waits for anything but its own input
        // vectors.
        // With few rows a thread-block cluster shares every row of its chunks, as in the one-shot exchange.
        const int cl = cluster_size(), cr = cluster_cta_rank();
        const int ncl = nb / cl, cid = vb / cl;
        const int nk = cid < nchunks ? (nchunks - cid + ncl - 1) / ncl : 0;
        auto r0_of = [&](int k) { return (cid + k * ncl) * R; };
        auto r1_of = [&](int k) { const int r1 = (cid + k * ncl) * R + R; return r1 < p.rows ? r1 : p.rows; };
        // a lead beyond the CTA's own chunks means "finish the earlier role first"
        const int lp = p.lead_push < nk ? p.lead_push : nk, lr = p.lead_reduce < nk ? p.lead_reduce : nk;
        const int steps = nk > 0 ? nk + lp + lr : 0;
        for (int s = 0; s < steps; ++s) {
            const int kr = s - lp, kf = kr - lr;
            const bool do_a = s < nk, do_b = kr >= 0 && kr < nk, do_c = kf >= 0 && kf < nk;
            for (int rr = 0; rr < R; ++rr) {
                const int ra = do_a && r0_of(s) + rr < r1_of(s) ? r0_of(s) + rr : -1;
                const int rb = do_b && r0_of(kr) + rr < r1_of(kr) ? r0_of(kr) + rr : -1;
                const int rc = do_c && r0_of(kf) + rr < r1_of(kf) ? r0_of(kf) + rr : -1;
                if (ra >= 0 || rb >= 0 || rc >= 0)
                    two_shot_step<T, NR, VPT, FUSED>(p, ts, ra, rb, rc, cr, cl, sm, parity, static_scale);
            }
        }
    } else {
        // one-shot: every rank receives every other rank's whole row and reduces it locally.  A
        // row belongs to a cluster of CTAs, each of which exchanges and finishes one segment.
        const int cl = cluster_size(), cr = cluster_cta_rank();
        const int ncl = nb / cl, cid = vb / cl;
        const int nk = cid < p.rows ? (p.rows - cid + ncl - 1) / ncl : 0;   // rows_per_chunk is 1 on this path
        const uint4 *in = reinterpret_cast<const uint4 *>(p.in);
        int64_t bo = 0;
        for (int k = 0; k < nk; ++k) {
            const int row = cid + k * ncl;
            const int len = row_len(p, row);
            RowSeg seg;
            seg.v0 = cr * p.seg_vecs;
            seg.v1 = seg.v0 + p.seg_vecs < len ? seg.v0 + p.seg_vecs : len;
            seg.cl_rank = cr;
            seg.cl_size = cl;
            const int64_t rbase = static_cast<int64_t>(row) * p.row_vecs;
            uint4 x[VPT], res[VPT];
#pragma unroll
            for (int i = 0; i < VPT; ++i) {
                const int v = seg.v0 + threadIdx.x + i * blockDim.x;
                x[i] = v < seg.v1 ? ld_stream(in + rbase + v) : make_uint4(0, 0, 0, 0);
            }
            if (k == 0) {
                // the counter is fetched while the first row's loads are in flight
                begin_call(st, nb, sm);
                __syncthreads();
                bo = p.os_off + static_cast<int64_t>(sm.seq & 1ull) * NR * p.os_slot_bytes;
            }
#pragma unroll
            for (int i = 0; i < VPT; ++i) {
                const int v = seg.v0 + threadIdx.x + i * blockDim.x;
                if (v < seg.v1) {
                    const uint4 send = payload<T>(x[i]);
#pragma unroll
                    for (int d = 1; d < NR; ++d) {
                        const int j = (p.rank + d) % NR;
                        st_peer(reinterpret_cast<uint4 *>(p.peer_data[j] + bo + p.rank * p.os_slot_bytes) + rbase + v, send);
                    }
                }
            }
            if constexpr (FUSED) load_residual<T, VPT>(p.ep, seg, row, whole_cta(), res);   // in flight while the peers' rows arrive
            char *mine = p.peer_data[p.rank] + bo;
#pragma unroll
            for (int i = 0; i < VPT; ++i) {
                const int v = seg.v0 + threadIdx.x + i * blockDim.x;
                if (v < seg.v1) {
                    uint4 part[NR];
#pragma unroll
                    for (int s = 0; s < NR; ++s)
                        part[s] = s == p.rank ? x[i] : ld_poll(reinterpret_cast<const uint4 *>(mine + s * p.os_slot_bytes) + rbase + v);
#pragma unroll
                    for (int s = 0; s < NR; ++s) {
                        if (s != p.rank) {
                            uint4 *addr = reinterpret_cast<uint4 *>(mine + s * p.os_slot_bytes) + rbase + v;
                            part[s] = wait_landed(addr, part[s], st, p.rank, kStageOneShot, s);
                            st_empty(addr);
                        }
                    }
                    x[i] = sum_in_rank_order<T, NR>(part);
                }
            }
            if constexpr (FUSED) {
                row_epilogue<T, VPT>(p.ep, seg, row, whole_cta(), x, res, sm, parity, static_scale);
                parity ^= 1;
            } else {
#pragma unroll
                for (int i = 0; i < VPT; ++i) {
                    const int v = seg.v0 + threadIdx.x + i * blockDim.x;
                    if (v < seg.v1) st_stream(reinterpret_cast<uint4 *>(p.out) + rbase + v, x[i]);
                }
            }
        }
        if (nk == 0) begin_call(st, nb, sm);   // a CTA without rows still takes its ticket
    }
}

// ---------------------------------------------------------------------------------------
// two-shot exchange with specialised warps (the bandwidth regime: more rows than SMs)
// ---------------------------------------------------------------------------------------
// One CTA per SM; CTA b of every rank owns rows b, b + gridDim, ...  Its warps split into three
// roles that each walk that row list on their own and meet only through the data:
//
//   scatter (ts threads)  reads the row of this rank's input and pushes slice j into slot
//                         `rank` of rank j, for every peer j.  Waits for nothing, so it runs
//                         ahead as far as NVLink lets it: the staging holds the whole message.
//   reduce  (tr threads)  for the slice this rank owns: polls the N - 1 slots, adds this rank's
//                         own slice straight from the input, sums in rank order in fp32, rounds
//                         once and pushes the result into every rank's gather area.
//   finish  (tf threads)  polls the gathered row, adds the residual and runs the epilogue (or,
//                         for the plain all-reduce, copies it out).
//
// Every transfer is a push of self-announcing vectors (common.cuh), so no role ever fences or
// signals; a role that waits for data only parks its own warps while the SM's schedulers run the
// others, which is what a single thread-set walking the three roles in lock step cannot do.  The
// row reductions of the finishing warps use a named barrier of their own.
template <typename T, int NR>
__device__ __forceinline__ void ws_scatter(const ArParams &p, int64_t ts_off, int vb, int nb, int tid, int nthreads,
                                           const volatile int *rows_finished) {
    constexpr int U = NR == 2 ? 4 : (NR == 4 ? 2 : 1);   // slice vectors per thread and peer that travel together
    const uint4 *in = reinterpret_cast<const uint4 *>(p.in);
    int k = 0;
    for (int row = vb; row < p.rows; row += nb, ++k) {
        // Stay within `scatter_lead` rows of the finishing warps: what is pushed further ahead would wait in
        // the peers' staging long enough to fall out of their L2 and come back from HBM.  The wait is on
        // shared memory and bounded (a stalled finisher must not stop the scatter for good).
        if (p.scatter_lead > 0) {
            for (int spin = 0; k - *rows_finished > p.scatter_lead && spin < (1 << 16); ++spin) __nanosleep(100);
        }
        const int len = row_len(p, row);
        const uint4 *src = in + static_cast<int64_t>(row) * p.row_vecs;
        const int64_t slot_row = static_cast<int64_t>(row) * p.vpr;
        if (p.ready) wait_ready(p.ready + row / p.ready_rows, p.ready_value, p.st, p.rank);
        for (int v0 = tid; v0 < p.vpr; v0 += U * nthreads) {
            uint4 a[NR - 1][U];
#pragma unroll
            for (int d = 1; d < NR; ++d) {
                const int j = (p.rank + d) % NR;
#pragma unroll
                for (int u = 0; u < U; ++u) {
                    const int vl = v0 + u * nthreads;
                    if (vl < p.vpr && j * p.vpr + vl < len) a[d - 1][u] = ld_stream(src + j * p.vpr + vl);
                }
            }
#pragma unroll
            for (int d = 1; d < NR; ++d) {
                const int j = (p.rank + d) % NR;
                uint4 *dst = reinterpret_cast<uint4 *>(p.peer_data[j] + ts_off + p.rank * p.rs_slot_bytes) + slot_row;
#pragma unroll
                for (int u = 0; u < U; ++u) {
                    const int vl = v0 + u * nthreads;
                    if (vl < p.vpr && j * p.vpr + vl < len) st_peer(dst + vl, payload<T>(a[d - 1][u]));
                }
            }
        }
    }
}

// Two ranks, one hop: the scattering threads push whole rows of this rank's input into the peer's gather area.
// With two ranks a two-shot exchange sends half of every row twice (the peer's slice, then the reduced own slice)
// and a whole row once is the same number of bytes, so the second hop and the slice reduction buy nothing.
template <typename T>
__device__ __forceinline__ void ws_push_rows(const ArParams &p, int64_t ag_ts, int vb, int nb, int tid, int nthreads,
                                             const volatile int *rows_finished) {
    constexpr int U = 4;
    const uint4 *in = reinterpret_cast<const uint4 *>(p.in);
    uint4 *peer = reinterpret_cast<uint4 *>(p.ag_base[p.rank ^ 1] + ag_ts);
    int k = 0;
    for (int row = vb; row < p.rows; row += nb, ++k) {
        if (p.scatter_lead > 0) {   // as in ws_scatter: what waits too long in the peer's staging falls out of its L2
            for (int spin = 0; k - *rows_finished > p.scatter_lead && spin < (1 << 16); ++spin) __nanosleep(100);
        }
        const int len = row_len(p, row);
        const int64_t base = static_cast<int64_t>(row) * p.row_vecs;
        for (int v0 = tid; v0 < len; v0 += U * nthreads) {
            uint4 a[U];
#pragma unroll
            for (int u = 0; u < U; ++u)
                if (v0 + u * nthreads < len) a[u] = ld_stream(in + base + v0 + u * nthreads);
#pragma unroll
            for (int u = 0; u < U; ++u)
                if (v0 + u * nthreads < len) st_peer(peer + base + v0 + u * nthreads, payload<T>(a[u]));
        }
    }
}

template <typename T, int NR>
__device__ __forceinline__ void ws_reduce(const ArParams &p, int64_t ts_off, int64_t ag_ts, int vb, int nb, int tid, int nthreads) {
    constexpr int U = NR == 2 ? 4 : (NR == 4 ? 2 : 1);   // slice vectors per thread in flight together: U * NR loads
    const uint4 *in = reinterpret_cast<const uint4 *>(p.in);
    char *mine = p.peer_data[p.rank] + ts_off;
    for (int row = vb; row < p.rows; row += nb) {
        const int len = row_len(p, row);
        const int64_t base = static_cast<int64_t>(row) * p.row_vecs + p.rank * p.vpr;
        const int64_t slot_row = static_cast<int64_t>(row) * p.vpr;
        if (p.ready) wait_ready(p.ready + row / p.ready_rows, p.ready_value, p.st, p.rank);   // this rank's own slice comes from `in`
        for (int v0 = tid; v0 < p.vpr; v0 += U * nthreads) {
            uint4 part[U][NR];
            bool have[U];
#pragma unroll
            for (int u = 0; u < U; ++u) {
                const int vl = v0 + u * nthreads;
                have[u] = vl < p.vpr && p.rank * p.vpr + vl < len;
                if (have[u]) {
#pragma unroll
                    for (int s2 = 0; s2 < NR; ++s2)
                        part[u][s2] = s2 == p.rank ? ld_stream(in + base + vl)
                                                   : ld_poll(reinterpret_cast<const uint4 *>(mine + s2 * p.rs_slot_bytes) + slot_row + vl);
                }
            }
#pragma unroll
            for (int u = 0; u < U; ++u) {
                if (have[u]) {
                    const int vl = v0 + u * nthreads;
#pragma unroll
                    for (int s2 = 0; s2 < NR; ++s2) {
                        if (s2 != p.rank) {
                            uint4 *addr = reinterpret_cast<uint4 *>(mine + s2 * p.rs_slot_bytes) + slot_row + vl;
                            part[u][s2] = wait_landed(addr, part[u][s2], p.st, p.rank, kStageScatter, s2);
                            st_empty(addr);
                        }
                    }
                    const uint4 red = payload<T>(sum_in_rank_order<T, NR>(part[u]));
                    if (p.ag_mc) {
                        // the switch copies this one store into every rank's gather area, this rank's included
                        multimem_st(reinterpret_cast<uint4 *>(p.ag_mc + ag_ts) + base + vl, red);
                    } else {
#pragma unroll
                        for (int d = 0; d < NR; ++d) {
                            const int j = (p.rank + d) % NR;   // start with myself, then fan out: spreads the links
                            st_peer(reinterpret_cast<uint4 *>(p.ag_base[j] + ag_ts) + base + vl, red);
                        }
                    }
                }
            }
        }
    }
}

// OWN (two ranks, one hop): the gather area holds the peer's row, not the sum; this rank's own row is read from
// its input and the two are added in rank order, in fp32, rounded once.
template <typename T, int VPT, bool FUSED, bool FULL, bool OWN = false>
__device__ __forceinline__ void ws_finish(const ArParams &p, int64_t ag_ts, int vb, int nb, const Group &grp, EpilogueSmem &sm) {
    // With up to two vectors per thread the loads of the NEXT row (first poll of the gathered row, residual)
    // are issued before the current row's epilogue, so a row's arithmetic hides the next row's memory latency.
    constexpr bool AHEAD = VPT <= 2;
    const uint4 *in = reinterpret_cast<const uint4 *>(p.in);
    float static_scale = 1.f;
    if constexpr (FUSED) {
        if (p.ep.q.mode == kQuantStatic) static_scale = *p.ep.scale_out;
    }
    uint4 *ag = reinterpret_cast<uint4 *>(p.ag_base[p.rank] + ag_ts);
    int parity = 0, done = 0;
    uint4 x[VPT], res[VPT], own[OWN ? VPT : 1], nx[AHEAD ? VPT : 1], nres[AHEAD ? VPT : 1], nown[AHEAD && OWN ? VPT : 1];
    auto issue = [&](int row, uint4 (&dx)[AHEAD ? VPT : 1], uint4 (&dres)[AHEAD ? VPT : 1], uint4 (&down)[AHEAD && OWN ? VPT : 1]) {
        if constexpr (AHEAD) {
            const int len = row < p.rows ? row_len(p, row) : 0;
            const int64_t base = static_cast<int64_t>(row) * p.row_vecs;
#pragma unroll
            for (int i = 0; i < VPT; ++i) {
                const int v = grp.tid + i * grp.n;
                const bool inside = FULL ? row < p.rows : v < len;
                dx[i] = inside ? ld_poll(ag + base + v) : make_uint4(0, 0, 0, 0);
                if constexpr (FUSED) dres[i] = inside ? ld_stream(reinterpret_cast<const uint4 *>(p.ep.residual) + base + v) : make_uint4(0, 0, 0, 0);
                if constexpr (OWN) down[i] = inside ? ld_stream(in + base + v) : make_uint4(0, 0, 0, 0);
            }
        }
    };
    if constexpr (AHEAD) issue(vb, nx, nres, nown);
    for (int row = vb; row < p.rows; row += nb) {
        const int len = row_len(p, row);
        const int64_t base = static_cast<int64_t>(row) * p.row_vecs;
        const RowSeg seg = RowSeg{0, len, 0, 1};
        if constexpr (AHEAD) {
#pragma unroll
            for (int i = 0; i < VPT; ++i) {
                x[i] = nx[i];
                res[i] = nres[i];
                if constexpr (OWN) own[i] = nown[i];
            }
            issue(row + nb, nx, nres, nown);
        } else {
#pragma unroll
            for (int i = 0; i < VPT; ++i) {
                const int v = grp.tid + i * grp.n;
                x[i] = (FULL || v < len) ? ld_poll(ag + base + v) : make_uint4(0, 0, 0, 0);
                if constexpr (OWN) own[i] = (FULL || v < len) ? ld_stream(in + base + v) : make_uint4(0, 0, 0, 0);
            }
            if constexpr (FUSED) load_residual<T, VPT, FULL>(p.ep, seg, row, grp, res);
        }
#pragma unroll
        for (int i = 0; i < VPT; ++i) {
            const int v = grp.tid + i * grp.n;
            if (FULL || v < len) {
                x[i] = wait_landed(ag + base + v, x[i], p.st, p.rank, kStageGather, OWN ? (p.rank ^ 1) : v / p.vpr);
                st_empty(ag + base + v);
                if constexpr (OWN) {
                    const uint4 part[2] = {p.rank == 0 ? own[i] : x[i], p.rank == 0 ? x[i] : own[i]};
                    x[i] = sum_in_rank_order<T, 2>(part);
                }
            }
        }
        if constexpr (FUSED) {
            row_epilogue<T, VPT, FULL>(p.ep, seg, row, grp, x, res, sm, parity, static_scale);
            parity ^= 1;
        } else {
#pragma unroll
            for (int i = 0; i < VPT; ++i) {
                const int v = grp.tid + i * grp.n;
                if (FULL || v < len) st_stream(reinterpret_cast<uint4 *>(p.out) + base + v, x[i]);
            }
        }
        if (grp.tid == 0) *const_cast<volatile int *>(&sm.rows_finished) = ++done;
    }
}

template <typename T, int NR, int VPT, bool FUSED>
__device__ __forceinline__ void ar_ws_body(const ArParams &p, int vb, int nb, EpilogueSmem &sm) {
    if (cluster_size() != p.cluster) {   // this kernel is planned without clusters
        if (threadIdx.x == 0) record_status(p.st, kStatusClusterMismatch, p.rank, vb, kStageScatter, p.rank, cluster_size());
        return;
    }
    begin_call(p.st, nb, sm);
    if (threadIdx.x == 0) sm.rows_finished = 0;
    __syncthreads();
    const int64_t ts_off = static_cast<int64_t>(sm.seq & 1ull) * p.ts_stride;
    const int64_t ag_ts = static_cast<int64_t>(sm.seq & 1ull) * p.ag_stride;
    const int tid = threadIdx.x;
    if (tid < p.tf) {
        const Group grp{tid, p.tf, 1};
        if (p.full) ws_finish<T, VPT, FUSED, true>(p, ag_ts, vb, nb, grp, sm);
        else ws_finish<T, VPT, FUSED, false>(p, ag_ts, vb, nb, grp, sm);
    } else if (tid < p.tf + p.tr) {
        ws_reduce<T, NR>(p, ts_off, ag_ts, vb, nb, tid - p.tf, p.tr);
    } else {
        ws_scatter<T, NR>(p, ts_off, vb, nb, tid - p.tf - p.tr, p.ts, &sm.rows_finished);
    }
}

constexpr int kWsMaxThreads = 768;   // 512 finishing + 128 reducing + 128 scattering threads: one CTA per SM

template <typename T, int NR, int VPT, bool FUSED>
__global__ void __launch_bounds__(kWsMaxThreads, 1)
    ar_ws_kernel(const __grid_constant__ ArParams p) {
    __shared__ EpilogueSmem sm;
    grid_dependency_sync();
    ar_ws_body<T, NR, VPT, FUSED>(p, blockIdx.x, gridDim.x, sm);
}

// N ranks in one launch on one GPU (see ar_emulated_kernel).
template <typename T, int NR, int VPT, bool FUSED>
__global__ void __launch_bounds__(kWsMaxThreads, 1)
    ar_ws_emulated_kernel(const ArParams *params_by_rank, int nb) {
    __shared__ EpilogueSmem sm;
    __shared__ ArParams p;
    const int rank = blockIdx.x / nb;
    for (int i = threadIdx.x; i < static_cast<int>(sizeof(ArParams) / 4); i += blockDim.x)
        reinterpret_cast<uint32_t *>(&p)[i] = reinterpret_cast<const uint32_t *>(params_by_rank + rank)[i];
    __syncthreads();
    ar_ws_body<T, NR, VPT, FUSED>(p, blockIdx.x % nb, nb, sm);
}

// Two ranks, one hop (see ws_push_rows): finishing warps that add their own row, and pushing warps.  A kernel of
// its own because it has no reducing warps: 640 threads leave the finishing warps 96 registers for the extra row.
constexpr int kWs1PushThreads = 128;
constexpr int kWs1MaxThreads = 512 + kWs1PushThreads;

template <typename T, int VPT>
__device__ __forceinline__ void ar_ws1_body(const ArParams &p, int vb, int nb, EpilogueSmem &sm) {
    if (cluster_size() != p.cluster) {   // this kernel is planned without clusters
        if (threadIdx.x == 0) record_status(p.st, kStatusClusterMismatch, p.rank, vb, kStageGather, p.rank, cluster_size());
        return;
    }
    begin_call(p.st, nb, sm);
    if (threadIdx.x == 0) sm.rows_finished = 0;
    __syncthreads();
    const int64_t ag_ts = static_cast<int64_t>(sm.seq & 1ull) * p.ag_stride;
    const int tid = threadIdx.x;
    if (tid < p.tf) {
        const Group grp{tid, p.tf, 1};
        if (p.full) ws_finish<T, VPT, true, true, true>(p, ag_ts, vb, nb, grp, sm);
        else ws_finish<T, VPT, true, false, true>(p, ag_ts, vb, nb, grp, sm);
    } else {
        ws_push_rows<T>(p, ag_ts, vb, nb, tid - p.tf, p.ts, &sm.rows_finished);
    }
}

template <typename T, int VPT>
__global__ void __launch_bounds__(kWs1MaxThreads, 1)
    ar_ws1_kernel(const __grid_constant__ ArParams p) {
    __shared__ EpilogueSmem sm;
    grid_dependency_sync();
    ar_ws1_body<T, VPT>(p, blockIdx.x, gridDim.x, sm);
}

// The two ranks in one launch on one GPU (see ar_emulated_kernel).
template <typename T, int VPT>
__global__ void __launch_bounds__(kWs1MaxThreads, 1)
    ar_ws1_emulated_kernel(const ArParams *params_by_rank, int nb) {
    __shared__ EpilogueSmem sm;
    __shared__ ArParams p;
    const int rank = blockIdx.x / nb;
    for (int i = threadIdx.x; i < static_cast<int>(sizeof(ArParams) / 4); i += blockDim.x)
        reinterpret_cast<uint32_t *>(&p)[i] = reinterpret_cast<const uint32_t *>(params_by_rank + rank)[i];
    __syncthreads();
    ar_ws1_body<T, VPT>(p, blockIdx.x % nb, nb, sm);
}

// ---------------------------------------------------------------------------------------
// N GPUs, bandwidth regime, through symmetric memory and the NVSwitch
// ---------------------------------------------------------------------------------------
// Every rank owns a buffer with the same layout (input copy | reduced tensor | flags), mapped
// by all ranks and, with MC, also behind one multicast address.  For a chunk of rows, CTA b of
// every rank
//   1. copies its rows of the rank's input into its own buffer and raises flag[0][b][rank] on
//      all ranks;
//   2. once all N flags of the chunk are up, reduces the column slice this rank owns: with MC
//      one multimem load per 16 bytes returns the sum over all ranks, added in the switch, and
//      one multimem store writes it to every rank's reduced tensor; without MC the slice is
//      read from every rank's buffer, summed in rank order and stored rank by rank.  Then
//      raises flag[1][b][rank] on all ranks;
//   3. once all N of those are up, runs the epilogue on whole rows of its own reduced tensor.
// With MC a GPU sends and receives S(1 + 1/N) bytes per direction for a message of S bytes,
// where the push exchange moves 2S(N-1)/N: 1.56x less at N = 8.
// Flags carry (call number << 20 | chunk + 1) and only grow, so nothing is ever reset, and the
// buffers need no double buffering: a rank's kernel ends only after every peer has raised the
// stage-2 flags of all chunks, i.e. after every peer has finished reading this rank's input
// copy; and a peer's stage-2 stores of the next call wait for this rank's stage-1 flag of the
// next call.  The three steps of consecutive chunks are staggered as in the push exchange.
constexpr int kSymFlagStages = 2;
constexpr int64_t kSymFlagBytes = static_cast<int64_t>(kSymFlagStages) * kMaxBlocks * kMaxRanks * 8;

template <typename T>
__device__ __noinline__ void sym_stage_in(const ArParams &p, int r0, int r1) {
    constexpr int U = 4;
    const uint4 *in = reinterpret_cast<const uint4 *>(p.in);
    uint4 *dst = reinterpret_cast<uint4 *>(p.sym[p.rank] + p.sym_in_off);
    const int64_t v_begin = static_cast<int64_t>(r0) * p.row_vecs, v_end = static_cast<int64_t>(r1) * p.row_vecs;
    const int B = blockDim.x;
    for (int64_t v0 = v_begin + threadIdx.x; v0 < v_end; v0 += U * B) {
        uint4 val[U];
#pragma unroll
        for (int u = 0; u < U; ++u)
            if (v0 + u * B < v_end) val[u] = ld_stream(in + v0 + u * B);
#pragma unroll
        for (int u = 0; u < U; ++u)
            if (v0 + u * B < v_end) st_peer(dst + v0 + u * B, val[u]);
    }
}

template <typename T, int NR, bool MC>
__device__ __noinline__ void sym_reduce_bcast(const ArParams &p, int r0, int r1) {
    constexpr int IB = MC ? 4 : (NR >= 8 ? 1 : (NR == 4 ? 2 : 4));
    const int items = (r1 - r0) * p.vpr;
    const int B = blockDim.x;
    for (int it0 = threadIdx.x; it0 < items; it0 += IB * B) {
        int64_t off[IB];
        uint4 red[IB];
        uint4 part[MC ? 1 : IB][MC ? 1 : NR];
#pragma unroll
        for (int b = 0; b < IB; ++b) {
            const int it = it0 + b * B;
            off[b] = -1;
            if (it < items) {
                const int rr = it / p.vpr;
                const int v = p.rank * p.vpr + (it - rr * p.vpr);
                if (v < p.row_vecs) {
                    off[b] = (static_cast<int64_t>(r0 + rr) * p.row_vecs + v) * 16;
                    if constexpr (MC) {
                        red[b] = multimem_ld_sum<T>(p.sym_mc + p.sym_in_off + off[b]);
                    } else {
#pragma unroll
                        for (int s = 0; s < NR; ++s) part[b][s] = ld_poll(p.sym[s] + p.sym_in_off + off[b]);
                    }
                }
            }
        }
#pragma unroll
        for (int b = 0; b < IB; ++b) {
            if (off[b] >= 0) {
                if constexpr (MC) {
                    multimem_st(p.sym_mc + p.sym_out_off + off[b], red[b]);
                } else {
                    const uint4 r = sum_in_rank_order<T, NR>(part[b]);
#pragma unroll
                    for (int d = 0; d < NR; ++d) st_peer(p.sym[(p.rank + d) % NR] + p.sym_out_off + off[b], r);
                }
            }
        }
    }
}

template <typename T, int VPT>
__device__ __noinline__ void sym_finish_rows(const ArParams &p, int r0, int r1, EpilogueSmem &sm, int &parity, float static_scale) {
    const uint4 *out = reinterpret_cast<const uint4 *>(p.sym[p.rank] + p.sym_out_off);
    const RowSeg seg = whole_row(p.row_vecs);
    for (int row = r0; row < r1; ++row) {
        const int64_t base = static_cast<int64_t>(row) * p.row_vecs;
        uint4 x[VPT], res[VPT];
#pragma unroll
        for (int i = 0; i < VPT; ++i) {
            const int v = threadIdx.x + i * blockDim.x;
            x[i] = v < p.row_vecs ? ld_staging(out + base + v) : make_uint4(0, 0, 0, 0);
        }
        load_residual<T, VPT>(p.ep, seg, row, whole_cta(), res);
        row_epilogue<T, VPT>(p.ep, seg, row, whole_cta(), x, res, sm, parity, static_scale);
        parity ^= 1;
    }
}

template <typename T, int NR, int VPT, bool MC>
__device__ __forceinline__ void ar_sym_body(const ArParams &p, int vb, int nb, EpilogueSmem &sm) {
    LocalState *st = p.st;
    const float static_scale = p.ep.q.mode == kQuantStatic ? *p.ep.scale_out : 1.f;
    begin_call(st, nb, sm);
    __syncthreads();
    const unsigned long long call = sm.seq;
    const int R = p.rows_per_chunk;
    const int nchunks = (p.rows + R - 1) / R;
    const int nk = vb < nchunks ? (nchunks - vb + nb - 1) / nb : 0;
    auto r0_of = [&](int k) { return (vb + k * nb) * R; };
    auto r1_of = [&](int k) { const int r1 = (vb + k * nb) * R + R; return r1 < p.rows ? r1 : p.rows; };
    auto flag_index = [&](int stage, int src) { return (static_cast<int64_t>(stage) * kMaxBlocks + vb) * kMaxRanks + src; };
    auto tag = [&](int k) { return (call << 20) | static_cast<unsigned long long>(k + 1); };
    // publish: everything this CTA has written so far is visible to a rank that sees the flag
    auto raise = [&](int stage, int k) {
        __syncthreads();
        if (threadIdx.x == 0) {
            __threadfence_system();
            const int64_t idx = flag_index(stage, p.rank);
            if constexpr (MC) {
                multimem_st_flag_release(reinterpret_cast<unsigned long long *>(p.sym_mc + p.sym_flag_off) + idx, tag(k));
            } else {
#pragma unroll
                for (int j = 0; j < NR; ++j)
                    st_flag_release(reinterpret_cast<unsigned long long *>(p.sym[j] + p.sym_flag_off) + idx, tag(k));
            }
        }
    };
    auto await = [&](int stage, int k) {
        if (threadIdx.x < NR)
            wait_flag(reinterpret_cast<const unsigned long long *>(p.sym[p.rank] + p.sym_flag_off) + flag_index(stage, threadIdx.x),
                      tag(k), st, p.rank, stage == 0 ? kStageSymIn : kStageSymOut, threadIdx.x);
        __syncthreads();
    };
    int parity = 0;
    const int steps = nk > 0 ? nk + 2 : 0;
    for (int s = 0; s < steps; ++s) {
        if (s < nk) {
            sym_stage_in<T>(p, r0_of(s), r1_of(s));
            raise(0, s);
        }
        const int kr = s - 1;
        if (kr >= 0 && kr < nk) {
            await(0, kr);
            sym_reduce_bcast<T, NR, MC>(p, r0_of(kr), r1_of(kr));
            raise(1, kr);
        }
        const int kf = s - 2;
        if (kf >= 0 && kf < nk) {
            await(1, kf);
            sym_finish_rows<T, VPT>(p, r0_of(kf), r1_of(kf), sm, parity, static_scale);
        }
    }
}

template <typename T, int NR, int VPT, bool MC>
__global__ void __launch_bounds__(tile_max_threads<VPT>(), ar_min_blocks<VPT>())
    ar_sym_kernel(const __grid_constant__ ArParams p) {
    __shared__ EpilogueSmem sm;
    grid_dependency_sync();
    ar_sym_body<T, NR, VPT, MC>(p, blockIdx.x, gridDim.x, sm);
}

// The same for N ranks inside one launch on one GPU (peer loads instead of the multicast).
template <typename T, int NR, int VPT>
__global__ void __launch_bounds__(tile_max_threads<VPT>(), ar_min_blocks<VPT>())
    ar_sym_emulated_kernel(const ArParams *params_by_rank, int nb) {
    __shared__ EpilogueSmem sm;
    __shared__ ArParams p;
    const int rank = blockIdx.x / nb;
    for (int i = threadIdx.x; i < static_cast<int>(sizeof(ArParams) / 4); i += blockDim.x)
        reinterpret_cast<uint32_t *>(&p)[i] = reinterpret_cast<const uint32_t *>(params_by_rank + rank)[i];
    __syncthreads();
    ar_sym_body<T, NR, VPT, false>(p, blockIdx.x % nb, nb, sm);
}

template <typename T, int NR, int VPT, bool TWO_SHOT, bool FUSED>
__global__ void __launch_bounds__(ar_max_threads<VPT, TWO_SHOT>(), ar_resident_blocks<VPT, TWO_SHOT>())
    ar_kernel(const __grid_constant__ ArParams p) {
    __shared__ EpilogueSmem sm;
    grid_dependency_sync();
    ar_body<T, NR, VPT, TWO_SHOT, FUSED>(p, blockIdx.x, gridDim.x, sm);
}

// N ranks in one cooperative launch on one GPU: block b plays CTA (b % nb) of rank (b / nb).
// All blocks are co-resident (cooperative launch), so the flag waits between "ranks" are safe.
template <typename T, int NR, int VPT, bool TWO_SHOT, bool FUSED>
__global__ void __launch_bounds__(ar_max_threads<VPT, TWO_SHOT>(), ar_resident_blocks<VPT, TWO_SHOT>())
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

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
    EpilogueArgs ep;
};

template <typename T, int VPT>
__global__ void __launch_bounds__(tile_max_threads<VPT>(), tile_min_blocks<VPT>())
    fused_norm_quant_kernel(const __grid_constant__ NormQuantParams p) {
    __shared__ EpilogueSmem sm;
    grid_dependency_sync();
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
        const RowSeg seg = whole_row(p.ep.row_vecs);
        load_residual<T, VPT>(p.ep, seg, row, res);
        row_epilogue<T, VPT>(p.ep, seg, row, x, res, sm, parity, static_scale);
    }
}

// The same operation for many rows: persistent CTAs take rows blockIdx.x, + gridDim.x, ... and
// fetch each row (input and residual, contiguous in global memory) into a ring of STAGES
// shared-memory stages with two bulk copies that one thread issues.  A stage is refilled with
// the row STAGES ahead as soon as every thread has taken its vectors out of it, so the loads of
// the next rows are in flight during both block reductions of the current one.
// Dynamic shared memory: STAGES * 2 * row_vecs * 16 bytes.  Needs at least two warps per CTA
// (the refill relies on the block barrier inside the first reduction).
template <int VPT>
constexpr int staged_min_blocks() { return VPT == 4 ? 3 : (VPT == 8 ? 1 : (VPT == 2 ? 1 : 1)); }

template <typename T, int VPT, int STAGES>
__global__ void __launch_bounds__(tile_max_threads<VPT>(), staged_min_blocks<VPT>())
    fused_norm_quant_staged_kernel(const __grid_constant__ NormQuantParams p) {
    extern __shared__ __align__(128) unsigned char stage_mem[];
    __shared__ EpilogueSmem sm;
    __shared__ __align__(8) uint64_t full[STAGES];
    grid_dependency_sync();
    const uint32_t row_bytes = static_cast<uint32_t>(p.ep.row_vecs) * 16u;
    const int64_t nk = blockIdx.x < p.rows ? (p.rows - blockIdx.x + gridDim.x - 1) / gridDim.x : 0;
    auto issue = [&](int64_t k) {
        const int s = static_cast<int>(k % STAGES);
        const int64_t row = blockIdx.x + k * gridDim.x;
        unsigned char *dst = stage_mem + static_cast<size_t>(s) * 2 * row_bytes;
        mbar_expect_bytes(&full[s], 2 * row_bytes);
        bulk_load(dst, static_cast<const unsigned char *>(p.in) + row * row_bytes, row_bytes, &full[s]);
        bulk_load(dst + row_bytes, static_cast<const unsigned char *>(p.ep.residual) + row * row_bytes, row_bytes, &full[s]);
    };
    if (threadIdx.x == 0) {
#pragma unroll
        for (int s = 0; s < STAGES; ++s) mbar_init(&full[s], 1);
        mbar_init_fence();
        for (int64_t k = 0; k < STAGES && k < nk; ++k) issue(k);
    }
    __syncthreads();
    const float static_scale = p.ep.q.mode == kQuantStatic ? *p.ep.scale_out : 1.f;
    const RowSeg seg = whole_row(p.ep.row_vecs);
    for (int64_t k = 0; k < nk; ++k) {
        const int s = static_cast<int>(k % STAGES);
        mbar_wait(&full[s], static_cast<uint32_t>(k / STAGES) & 1u);
        const uint4 *sx = reinterpret_cast<const uint4 *>(stage_mem + static_cast<size_t>(s) * 2 * row_bytes);
        const uint4 *sr = sx + p.ep.row_vecs;
        uint4 x[VPT], res[VPT];
#pragma unroll
        for (int i = 0; i < VPT; ++i) {
            const int v = threadIdx.x + i * blockDim.x;
            x[i] = v < p.ep.row_vecs ? sx[v] : make_uint4(0, 0, 0, 0);
            res[i] = v < p.ep.row_vecs ? sr[v] : make_uint4(0, 0, 0, 0);
        }
        row_epilogue<T, VPT>(p.ep, seg, blockIdx.x + k * gridDim.x, x, res, sm, static_cast<int>(k & 1), static_scale,
                             [&] { if (threadIdx.x == 0 && k + STAGES < nk) issue(k + STAGES); });
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
    int rows_per_chunk;    // rows a CTA moves through one stage before it turns to the next stage
    int seg_vecs;          // vectors of a row held by one CTA of the cluster that owns the row (all of them without a cluster)
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
        if (row_c >= 0) load_residual<T, VPT>(p.ep, seg, row_c, res);
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
            row_epilogue<T, VPT>(p.ep, seg, row_c, x, res, sm, parity, static_scale);
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
            if constexpr (FUSED) load_residual<T, VPT>(p.ep, seg, row, res);   // in flight while the peers' rows arrive
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
                row_epilogue<T, VPT>(p.ep, seg, row, x, res, sm, parity, static_scale);
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
        load_residual<T, VPT>(p.ep, seg, row, res);
        row_epilogue<T, VPT>(p.ep, seg, row, x, res, sm, parity, static_scale);
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

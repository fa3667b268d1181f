/*
 * gpuk_b200 -- C ABI of the B200-native tensor-parallel epilogue
 * (all-reduce of per-rank partials + residual add + RMSNorm + FP8-e4m3 quantisation).
 *
 * Every entry point takes plain pointers and sizes, returns an int status (0 = success,
 * never throws, never aborts) and enqueues its GPU work on the CUDA stream it is given.
 * This is the boundary a binding for the reference's operator API links against; each
 * declaration names the reference interface it stands in for (paths are relative to the
 * reference project xytpai/gpuk).
 *
 * Threading: a workspace is not thread-safe and belongs to one process and one device
 * (same contract as the reference's CommWorkspace, src/ops/all_reduce_fusion.cpp:44-254).
 * All ranks of a group must issue the same sequence of collective calls with the same
 * shapes.  Calls on one workspace must be ordered on one stream.
 */
#ifndef GPUK_B200_H_
#define GPUK_B200_H_

#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

#define GPUK_IPC_HANDLE_BYTES 64 /* sizeof(cudaIpcMemHandle_t) */
#define GPUK_MAX_RANKS 8         /* src/common/communicator.h:57 */

/* status codes */
enum {
    GPUK_OK = 0,
    GPUK_ERR_INVALID_ARGUMENT = 1, /* bad rank / world size / null pointer / misaligned pointer */
    GPUK_ERR_CUDA = 2,             /* a CUDA runtime call failed; see gpuk_last_error() */
    GPUK_ERR_UNSUPPORTED = 3,      /* shape or dtype outside what the kernels cover */
    GPUK_ERR_NOT_READY = 4,        /* peers' memory has not been opened yet */
    GPUK_ERR_TOO_LARGE = 5,        /* message exceeds the workspace created by gpuk_ws_create */
    GPUK_ERR_PEER_TIMEOUT = 6,     /* a device-side wait for a peer ran out (gpuk_ws_status) */
    GPUK_ERR_BAD_LAUNCH = 7        /* a kernel found itself in another launch shape than planned (gpuk_ws_status) */
};

/* element types of the activations */
enum { GPUK_DTYPE_BF16 = 0, GPUK_DTYPE_F16 = 1, GPUK_DTYPE_F32 = 2 };

/*
 * quant_type of the fused operator.  0..2 keep the reference's meaning
 * (src/impl/all_reduce_fusion_impl.h:13-17, saturation values src/common/float8.h:216-218
 * and :249-251); 3 and 4 are additive.
 */
enum {
    GPUK_QUANT_NONE = 0,               /* norm_out has the input dtype */
    GPUK_QUANT_FP8_E4M3FN_240 = 1,     /* per-token dynamic scale = amax/240, e4m3fn codes */
    GPUK_QUANT_FP8_E4M3FNUZ_120 = 2,   /* per-token dynamic scale = amax/120, e4m3fnuz codes */
    GPUK_QUANT_FP8_E4M3FN_448 = 3,     /* per-token dynamic scale = amax/448, e4m3fn codes */
    GPUK_QUANT_FP8_E4M3FN_448_STATIC = 4 /* one caller-supplied scale: scale_out[0] is READ */
};

typedef struct gpuk_ws gpuk_ws; /* opaque; the reference passes it around as an int64 "fptr" */

/* Text of the most recent failure on the calling thread ("" if none). */
const char *gpuk_last_error(void);
const char *gpuk_status_string(int status);

/* ------------------------------------------------------------------------------------- */
/* workspace life cycle                                                                  */
/* ------------------------------------------------------------------------------------- */

/*
 * Replaces init_ar_fusion (src/register.cpp:5-6, src/ops/all_reduce_fusion.cpp:256-268) and
 * the CommWorkspace constructor (:46-70).  world_size must be 2, 4 or 8 and
 * 0 <= rank < world_size, otherwise GPUK_ERR_INVALID_ARGUMENT (the reference throws
 * std::invalid_argument).  max_size_in_bytes is the largest message (bytes of one rank's
 * input) the workspace must carry.  comm_ptrs_buf_len is accepted for signature
 * compatibility and ignored: no pointer table is needed because peers never read inputs.
 * Argument validation happens before any CUDA call.
 */
int gpuk_ws_create(int device_id, int rank, int world_size, int64_t max_size_in_bytes,
                   int64_t comm_ptrs_buf_len, gpuk_ws **out);

/* Replaces destroy_ar_fusion (src/register.cpp:7-8, all_reduce_fusion.cpp:270-273). */
int gpuk_ws_destroy(gpuk_ws *ws);

/*
 * Replace get_ar_fusion_barrier_handle / get_ar_fusion_data_handle (src/register.cpp:10-13,
 * all_reduce_fusion.cpp:275-283): write the 64-byte cudaIpcMemHandle_t of the flag array /
 * of the staging memory to `out`.  The exchange here needs no flags (data announces itself),
 * so the flag array is a small reserved allocation; its handle is still exported and opened
 * so that the reference's bootstrap sequence runs unchanged.
 */
int gpuk_ws_get_barrier_handle(gpuk_ws *ws, uint8_t out[GPUK_IPC_HANDLE_BYTES]);
int gpuk_ws_get_data_handle(gpuk_ws *ws, uint8_t out[GPUK_IPC_HANDLE_BYTES]);

/*
 * Replace open_ar_fusion_barrier_handles / open_ar_fusion_data_handles (src/register.cpp:15-18,
 * all_reduce_fusion.cpp:285-293, ipc_details::open_handles :15-34).  `handles` holds
 * world_size consecutive 64-byte handles in rank order; the entry of this rank is ignored.
 */
int gpuk_ws_open_barrier_handles(gpuk_ws *ws, const uint8_t *handles, int n);
int gpuk_ws_open_data_handles(gpuk_ws *ws, const uint8_t *handles, int n);

/*
 * Single-process alternative to the IPC exchange, for a process that owns all GPUs and has
 * enabled peer access itself -- the harness style of the reference's C++ tests
 * (test/cpp/test_all_reduce.cpp:337-356 with src/common/communicator.h:40-55).
 * gpuk_ws_local_pointers returns this rank's flag array and staging base;
 * gpuk_ws_set_peer_pointers installs all ranks' pointers (rank order) on this workspace.
 */
int gpuk_ws_local_pointers(gpuk_ws *ws, void **flags, void **data);
int gpuk_ws_set_peer_pointers(gpuk_ws *ws, void *const *flags, void *const *data, int n);
/*
 * Optional second exchange for the bandwidth regime, through symmetric memory: `bases[r]` is
 * rank r's buffer of `bytes` bytes as mapped in this process (same size on every rank, 256-byte
 * aligned; bases[rank] is this rank's own) and `mc_base` the NVSwitch multicast mapping of the
 * same buffers, or NULL.  The caller allocates and maps them (for one process per GPU e.g. with
 * torch.distributed._symmetric_memory, which is how GPUKDistEnv does it) and keeps them alive
 * while the workspace exists; the last 256 KiB hold flags and must be zero on every rank before
 * the first call.  With a multicast mapping the reduction runs inside the switch
 * (multimem.ld_reduce) and a GPU moves S(1 + 1/N) bytes per direction instead of 2S(N-1)/N;
 * the switch rounds the 16-bit sum in its own way (measured on B200: ties away from zero, so
 * about 15 % of the sums differ from round-to-nearest-even by one unit in the last place),
 * which is outside this library's parity bars: option "sym_multicast" = 0 keeps the exchange
 * but reads the peers' buffers with plain loads and sums in rank order, bit-exact.
 * Fused calls whose message is at least the option "sym_min_bytes" (default: never) and fits
 * (bytes - 256 KiB) / 2 take this exchange.  The reference has no counterpart (it pulls from
 * IPC-registered inputs, all_reduce_fusion.cpp:105-137).
 */
int gpuk_ws_attach_symmetric(gpuk_ws *ws, void *const *bases, int n, void *mc_base, int64_t bytes);

/* Replaces enable_p2p (src/common/communicator.h:40-55): peer access among devices 0..n-1. */
int gpuk_enable_peer_access(int n_devices);

/* ------------------------------------------------------------------------------------- */
/* graph-capture registration surface (kept for drop-in compatibility)                   */
/* ------------------------------------------------------------------------------------- */

/*
 * The reference registers input tensors seen during CUDA-graph capture so that peers can
 * read them in place (all_reduce_fusion.cpp:105-137, 168-233).  This implementation pushes
 * data and never reads a peer's input, so a captured call needs no registration: the
 * captured list is always empty and these calls succeed without effect.  They replace
 * ar_fusion_capture_clear (:295-298), get_ar_fusion_captured_handles / _offsets (:310-318)
 * and open_ar_fusion_captured_handles (:320-323).
 */
int gpuk_ws_capture_clear(gpuk_ws *ws);
int gpuk_ws_captured_count(gpuk_ws *ws, int *count);
int gpuk_ws_open_captured_handles(gpuk_ws *ws, const uint8_t *handles, const int64_t *offsets, int n,
                                  int64_t ptr_idx);
/*
 * Replace get_ar_fusion_tensor_handle / get_ar_fusion_tensor_offset (:300-308): the IPC
 * handle of the allocation that contains `ptr`, and ptr's byte offset inside it
 * (ipc_details::create_base_ptr, :36-40).
 */
int gpuk_tensor_ipc_handle(const void *ptr, uint8_t out[GPUK_IPC_HANDLE_BYTES]);
int gpuk_tensor_ipc_offset(const void *ptr, int64_t *offset);

/* ------------------------------------------------------------------------------------- */
/* the hot path                                                                          */
/* ------------------------------------------------------------------------------------- */

/*
 * Replaces allreduce_rms (src/register.cpp:35-40, all_reduce_fusion.cpp:363-396) and
 * allreduce_rms_fusion_impl (src/impl/all_reduce_fusion_impl.h:424-469).
 *
 *   allreduce_in [numel]            this rank's partial, contiguous, rows of `hidden`
 *   residual_in  [numel]            same on all ranks
 *   rms_gamma    [hidden]
 *   residual_out [numel]            = T(allreduce + residual)
 *   norm_out     [numel]            T, or FP8 bytes when quant_type != 0
 *   scale_out                       quant 1..3: [numel/hidden] fp32 written; quant 4: [1] fp32 read
 *
 * Any hidden that is a multiple of 16 bytes / element size up to 32768 elements (16-bit
 * types) is accepted (the reference: 1024, 2048, 4096 only, impl.h:389-401).  All device
 * pointers must be 16-byte aligned.  Asynchronous on `stream` (a cudaStream_t).
 */
int gpuk_allreduce_rms(gpuk_ws *ws, const void *allreduce_in, const void *residual_in,
                       const void *rms_gamma, void *residual_out, void *norm_out, float *scale_out,
                       int64_t numel, int hidden, int dtype, float eps, int quant_type, void *stream);

/*
 * The step before the path: the partial sums usually come out of the row-parallel GEMM
 * (model/tensor_parallel.py:112-123, F.linear at :117), which the reference lets finish before its
 * all-reduce starts.  Here the NEXT gpuk_allreduce_rms / gpuk_emulated_allreduce_rms call on `ws` may
 * start while its input is still being produced: word i of `ready` (device memory of this GPU, 4-byte
 * words) stands for rows [i * rows_per_word, (i + 1) * rows_per_word) of allreduce_in, and the kernel reads
 * a row only after its word has reached `value` (unsigned compare, so a producer can count calls up and
 * never reset the words).  The producer -- the epilogue of a row-block GEMM, a kernel behind it on its
 * stream, or a copy engine -- stores the word after the rows are complete; blocks may complete in any order.
 * Applies to one call and only where that call runs the two-shot exchange with specialised warps
 * (gpuk_plan.ws == 1), otherwise the call fails with GPUK_ERR_UNSUPPORTED and the caller orders it behind the
 * producer as usual.  A producer that needs SMs while the exchange runs must be given room: option
 * "ws_max_ctas" caps the SMs the exchange occupies.  A word that never arrives ends in the same bounded wait and
 * status report as a silent peer (stage 6).  ready = NULL clears a pending setting.
 * No counterpart in the reference.
 */
int gpuk_ws_set_ready_words(gpuk_ws *ws, const uint32_t *ready, int rows_per_word, uint32_t value);

/*
 * Replaces allreduce_inplace (src/register.cpp:33-34, all_reduce_fusion.cpp:340-361) and
 * allreduce_inplace_impl (impl.h:115-144): sum over ranks, fp32 accumulation in rank order,
 * one rounding, written back over `data`.  numel * element size must be a multiple of 16.
 */
int gpuk_allreduce_inplace(gpuk_ws *ws, void *data, int64_t numel, int dtype, void *stream);

/*
 * One GPU, no communication: residual add + RMSNorm + FP8 with `in` taking the place of
 * the all-reduced sum.  The reference has no such entry (GPUKDistEnv leaves fptr = None for
 * world_size 1, gpuk/__init__.py:72-73, and its fused call then fails); this is what the
 * Python wrapper dispatches to for a group of one.  Same argument meaning as
 * gpuk_allreduce_rms.
 */
int gpuk_residual_rms_quant(const void *in, const void *residual_in, const void *rms_gamma,
                            void *residual_out, void *norm_out, float *scale_out, int64_t numel,
                            int hidden, int dtype, float eps, int quant_type, void *stream);

/* ------------------------------------------------------------------------------------- */
/* policy, status, self-check                                                            */
/* ------------------------------------------------------------------------------------- */

/* How a call would be executed; pure host arithmetic, usable without a GPU. */
typedef struct gpuk_plan {
    int one_shot;       /* 1: one-shot exchange, 0: two-shot */
    int vpt;            /* 16-byte vectors of a row held per thread */
    int threads;        /* CTA size */
    int rows_per_chunk; /* rows a CTA takes through one pipeline role at a time (two-shot) */
    int grid;           /* CTAs per rank */
    int rows;
    int row_vecs;
    int64_t message_bytes;
    int cluster;        /* CTAs (one thread-block cluster) that share a row; 1 unless few rows must fill the GPU */
    int lead_push;      /* two-shot pipeline: chunks the scatter runs ahead of the reduction */
    int lead_reduce;    /* two-shot pipeline: chunks the reduction runs ahead of the epilogue */
    /* two-shot exchange without clusters: one CTA per SM whose warps are specialised (scatter / reduce /
     * finish); then grid is at most the SM count and the CTA has ws_tf + ws_tr + ws_ts threads */
    int ws;             /* 1: that kernel runs this call (vpt, threads, grid, rows_per_chunk above describe the other
                         * two-shot kernel, which the option "two_shot_ws" = 0 selects) */
    int ws_grid;        /* its CTAs per rank */
    int ws_vpt;         /* vectors of a row per finishing thread */
    int ws_tf, ws_tr, ws_ts; /* finishing / reducing / scattering threads per CTA */
} gpuk_plan;

/* force_mode values of gpuk_emulated_allreduce_rms */
#define GPUK_MODE_AUTO 0
#define GPUK_MODE_ONE_SHOT 1
#define GPUK_MODE_TWO_SHOT 2
#define GPUK_MODE_SYMMETRIC 3   /* through symmetric memory (gpuk_ws_attach_symmetric) */

/*
 * Launch plan for a message of `numel` elements in rows of `hidden` on `world_size` ranks.
 * ctas_per_sm_limit is the occupancy the caller assumes (<= 0: the built-in default),
 * oneshot_max_bytes the one-shot/two-shot crossover (<= 0: the built-in default per world
 * size; the reference's rule is impl.h:375-376).
 */
int gpuk_plan_allreduce_rms(int world_size, int64_t numel, int hidden, int dtype, int sm_count,
                            int ctas_per_sm_limit, int64_t oneshot_max_bytes, gpuk_plan *out);

/* Override the crossover (bytes of one rank's input; <= 0 restores the default). */
int gpuk_ws_set_oneshot_max_bytes(gpuk_ws *ws, int64_t bytes);
/*
 * Tuning options of the exchanges; all ranks must set the same values.  Names:
 * "rows_per_chunk" (rows a CTA takes through one pipeline role at a time, 0: default),
 * "ctas_per_sm" (cap on resident CTAs per SM, 0: default), "cluster" (CTAs of a thread-block
 * cluster that share a row: 1, 2, 4, 8, 0: default), "two_shot_ws" (1: two-shot calls without clusters run the
 * kernel with specialised warps, 0: the lock-step kernel), "two_rank_one_hop" (1, the default: at two ranks that
 * kernel pushes whole rows into the peer's staging and every rank adds its own row while finishing, one NVLink hop
 * for the bytes the two hops of reduce-scatter + all-gather would move; 0: two hops.  The fused call falls back to
 * two hops by itself when ready words are set or an output overlaps the input -- which, like everything about a
 * call, must be the same on every rank), "ws_finish_threads" / "ws_reduce_threads" /
 * "ws_scatter_threads" (its threads per role, 0: default), "ws_scatter_lead" (rows its scatter may run ahead of
 * its finish, -1: default, 0: unbounded), "ws_max_ctas" (SMs it may occupy, 0: all), "gather_multicast" (1: its
 * gather goes through the multicast address of the attached symmetric memory), "lead_push" / "lead_reduce" (pipeline
 * depths in chunks, 0: default), "oneshot_max_bytes", "sym_min_bytes" (smallest message that
 * takes the exchange through symmetric memory, 0: never), "sym_multicast" (1: reduce inside the
 * switch where a multicast mapping exists, 0: plain peer loads).  "test_withhold_cluster" = 1 is a
 * test hook: kernels are launched without their planned cluster attribute, which they must report
 * (status code 3) instead of writing partial rows.
 * The reference fixes these at compile time (communicator.h:57-58, impl.h:375-376).
 */
int gpuk_ws_set_option(gpuk_ws *ws, const char *name, int64_t value);
/*
 * Process-wide tuning of the one-GPU kernel behind gpuk_residual_rms_quant (which has no
 * workspace to carry options): "k1_stages" (shared-memory stages of the persistent variant: 2, 3,
 * 0 = never use it, -1 = default), "k1_staged_min_rows" (rows from which that variant runs,
 * -1 = default: more rows than the plain kernel has resident CTAs), "k1_ctas_per_sm" (cap on its
 * resident CTAs per SM, 0 = as many as fit).  One more name belongs to gpuk_fp8_linear_skinny:
 * "fp8_frags_per_warp" (16-row fragments a warp multiplies per k step: 1 = eight warps per CTA, 2 = four warps
 * that convert each activation vector once for two fragments; 0 = default: 2 for more than 16 tokens on at least 4096 output channels, else 1).
 * Not thread-safe against concurrent calls.
 */
int gpuk_set_tuning(const char *name, int64_t value);
/* Budget of every device-side wait for a peer, in nanoseconds (default 2 s). */
int gpuk_ws_set_timeout_ns(gpuk_ws *ws, uint64_t ns);

/*
 * Copies the workspace's device status words to `out` (synchronises the device):
 * out[0] = 0 ok / 1 wait timed out / 2 poll cap reached / 3 the kernel ran in a thread-block
 * cluster of another size than planned (out[6] = the size seen; it then wrote nothing and the
 * call returns GPUK_ERR_BAD_LAUNCH), out[1] = rank, out[2] = CTA,
 * out[3] = stage (0 one-shot, 1 scatter, 2 gather, 3 self-test, 4 / 5 the two flags of the
 * exchange through symmetric memory, 6 a ready word of this rank's own input), out[4] = peer whose data was
 * awaited, out[5] = thread, out[6] = word seen.  Returns GPUK_ERR_PEER_TIMEOUT if out[0] != 0.
 * The reference spins forever instead (communicator.h:98-99).
 */
int gpuk_ws_status(gpuk_ws *ws, uint32_t out[8]);
/*
 * Clears the status words and the abort latch and puts the staging memory back to its rest
 * state.  After a timeout every rank of the group must call this, with the device idle, before
 * the workspace is used again.
 */
int gpuk_ws_clear_status(gpuk_ws *ws);

/*
 * Self-check of the bounded wait: one thread waits, with the workspace's time budget, for
 * data that nothing sends, records the timeout and returns.  No fault, no hang; used by the
 * failure-detection test.
 */
int gpuk_ws_selftest_wait(gpuk_ws *ws, void *stream);

/*
 * The N-rank kernels run for all ranks inside ONE cooperative launch on the current GPU
 * (block b plays CTA b % grid of rank b / grid), against `world_size` workspaces created
 * on that GPU and wired together with gpuk_ws_set_peer_pointers.  For validating the
 * multi-rank logic where a single GPU is available.  Pointer arrays are indexed by rank;
 * for the plain all-reduce pass residual_in = NULL and hidden = 0 (then `allreduce_in[r]`
 * is reduced in place).  force_mode: 0 = policy decides, 1 = one-shot, 2 = two-shot.
 */
int gpuk_emulated_allreduce_rms(gpuk_ws *const *ws, int world_size, void *const *allreduce_in,
                                const void *residual_in, const void *rms_gamma, void *const *residual_out,
                                void *const *norm_out, float *const *scale_out, int64_t numel, int hidden,
                                int dtype, float eps, int quant_type, int force_mode, void *stream);

/*
 * The consumer of the fused operator's FP8 output for decode batches: out[m, n] (bf16) =
 * (x . w^T)[m, n] * x_scale[m] * w_scale[n], with x [m, k] and w [n, k] e4m3 (k contiguous), fp32
 * accumulation, one rounding.  x and x_scale are norm_out and scale_out of gpuk_allreduce_rms
 * (quant_type 3 or 1) as they are; w_scale holds one scale per output channel.  Replaces the F.linear that
 * follows the norm in model/tensor_parallel.py:66 (the reference has no FP8 path; a PyTorch caller would
 * otherwise use torch._scaled_mm).  Built for the weight-streaming regime: m <= 32 tokens
 * (GPUK_ERR_UNSUPPORTED beyond -- use a library GEMM there), n a multiple of 128, k a multiple of 64,
 * operands 16-byte aligned.  w_layout: 0 = w is [n, k] row-major as PyTorch holds it; 1 = w was rearranged once by
 * gpuk_fp8_pack_weight, so that the 16 rows x 64 bytes a warp multiplies at a time are one contiguous KiB and a
 * warp reads its rows as one sequential run of memory (rows that lie a power of two apart do not).  k_split = CTAs
 * of a thread-block cluster that share a tile of 128 output channels and split k (1, 2, 4, 8; 0: chosen from the
 * shape).  The sum order is fixed, so results are reproducible from call to call.
 */
int gpuk_fp8_linear_skinny(const void *x_fp8, const float *x_scale, const void *w_fp8, const float *w_scale,
                           void *out_bf16, int m, int n, int k, int w_layout, int k_split, void *stream);
/*
 * Rearranges FP8 weights [n, k] (row-major) into the blocked layout of w_layout = 1: block (n / 16, k / 64) holds
 * 16 rows x 64 bytes, row r at byte r * 64; the blocks of a 16-row band follow each other along k.  Done once per
 * weight matrix (the reference keeps its weights as nn.Linear does, model/tensor_parallel.py:62-67).  n a multiple
 * of 16, k of 64; `packed` holds n * k bytes and must not overlap w_fp8.
 */
int gpuk_fp8_pack_weight(const void *w_fp8, void *packed, int n, int k, void *stream);
/*
 * Synchronises the current device and returns GPUK_ERR_BAD_LAUNCH if a gpuk_fp8_linear_skinny launch on it
 * found itself in another thread-block cluster than planned (it then wrote nothing), else GPUK_OK.
 * Same contract as status 3 of gpuk_ws_status; the reference has no counterpart (impl.h launches no clusters).
 */
int gpuk_fp8_linear_status(void);

/*
 * No counterpart in the reference.  Same job as gpuk_emulated_allreduce_rms (fused op only)
 * for callers that must not allocate device memory -- a health probe or test harness inside a
 * process whose own arena already owns the GPU's memory, where a library-side cudaMalloc may
 * fail or disturb that arena.  It needs no workspaces: the staging memory is a fixed array
 * built into the library (about 8.5 MiB, held by every GPU that loads the library until the
 * process exits), which limits a message to 32 KiB per emulated rank (numel * element size);
 * larger requests return GPUK_ERR_TOO_LARGE.  Rows longer than 4096 16-byte vectors are not
 * built.  The first call on a device sets the array up and synchronises the stream: make it before
 * any stream capture (during a capture that first call is refused).  Later calls are stream-ordered
 * launches without a host synchronisation.  All calls on a device share the array, which keeps the
 * protocol's call counter between calls and is not cleared otherwise; calls that overlap on the GPU
 * race, so issue them one after another on one stream.  If a call gave up waiting (see
 * gpuk_selfcheck_status), the next call puts the array back to rest on the device before it starts.
 * Allocates nothing (no cudaMalloc, cudaFree or allocating library call).
 */
int gpuk_selfcheck_allreduce_rms(int world_size, void *const *allreduce_in, const void *residual_in,
                                 const void *rms_gamma, void *const *residual_out, void *const *norm_out,
                                 float *const *scale_out, int64_t numel, int hidden, int dtype, float eps,
                                 int quant_type, int force_mode, void *stream);
/*
 * No counterpart in the reference.  Waits for `stream` and copies the status words the last
 * gpuk_selfcheck_allreduce_rms call on the current device left (layout as gpuk_ws_status; the
 * first emulated rank that reported is returned): GPUK_OK, GPUK_ERR_PEER_TIMEOUT when a wait of
 * that call ran out (its outputs are then not valid), GPUK_ERR_BAD_LAUNCH when the kernel ran in
 * another cluster shape than planned.  Allocates nothing.
 */
int gpuk_selfcheck_status(uint32_t out[8], void *stream);

#ifdef __cplusplus
}
#endif
#endif /* GPUK_B200_H_ */

/*
 * liger_b200.h -- C ABI of the B200 (sm_100a) implementation of Liger's tensor-parallel
 * transformer-layer path.
 *
 * Every entry point is `extern "C"`, takes plain pointers and sizes, launches asynchronously on
 * the CUDA stream it is given (passed as void*, i.e. a cudaStream_t) and returns LIGER_OK or a
 * negative LIGER_ERR_* code; liger_last_error() gives the message for the calling thread.  All
 * tensors are fp16 (IEEE binary16) in device memory and row-major unless stated otherwise; all
 * accumulation is fp32.  There is no CPU fallback: without a CUDA device every compute entry
 * point fails with LIGER_ERR_CUDA.
 *
 * Citations of the form `src/...:lines` name the interface of the reference implementation
 * (MachineLearningSystem/24PPOPP-Liger) that the entry point replaces.
 */
#ifndef LIGER_B200_H
#define LIGER_B200_H

#include <stddef.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

#if defined(__GNUC__)
#define LIGER_API __attribute__((visibility("default")))
#else
#define LIGER_API
#endif

#define LIGER_OK 0
#define LIGER_ERR_INVALID (-1)     /* bad argument (shape, alignment, null pointer) */
#define LIGER_ERR_CUDA (-2)        /* a CUDA runtime / driver call failed */
#define LIGER_ERR_UNSUPPORTED (-3) /* shape outside what the kernels implement */
#define LIGER_ERR_DEVICE (-4)      /* the sticky device status word is set (a device-side wait timed out) */
#define LIGER_ERR_TOO_LARGE (-5)   /* a fixed-capacity resource is too small for the request */
#define LIGER_ERR_COMM (-6)        /* communicator set-up failed */

/* bits of the sticky device status word */
#define LIGER_DEV_TIMEOUT 1u /* a bounded device-side wait ran out */

/* Message describing the last error returned to the calling thread ("" if none). */
LIGER_API const char* liger_last_error(void);

/* Library version string. */
LIGER_API const char* liger_version(void);

/*
 * Sticky device status.  Kernels never trap or spin forever: a wait that exceeds its budget sets a bit
 * in a host-visible status word and the kernel unwinds.  (Shapes, strides, alignment and buffer extents are
 * checked on the host before a launch; kernels carry no index checks of their own.)
 * out[0] = LIGER_DEV_* bits, out[1] = location id, out[2..3] = detail.  Returns out[0].
 * The reference ignores every CUDA / cuBLAS / NCCL return code (e.g. src/layer/func_wrapper.h:25,42).
 */
LIGER_API int liger_device_status(unsigned int out[4]);
LIGER_API int liger_device_status_clear(void);
/*
 * How long a kernel of this library waits (on an mbarrier, a peer's flag, a barrier across ranks) before it
 * gives up, sets LIGER_DEV_TIMEOUT and unwinds: 2000 ms unless set here (for the current device) or through the
 * environment variable LIGER_WAIT_BUDGET_MS (every device).  The reference has no counterpart: its kernels
 * and NCCL's wait without limit (src/layer/func_wrapper.h:40-43).
 */
LIGER_API int liger_set_wait_budget_ms(int milliseconds);

/* ------------------------------------------------------------------------------------------ */
/* Seeded tensors (the reference leaves every buffer uninitialised: src/layer/linear.h:40,92,  */
/* src/layer/bert_layer.h:45,115-118, src/layer/operator.h:29-30, src/test_schedule.h:29-31)  */
/* ------------------------------------------------------------------------------------------ */

/*
 * dst[r*dst_ld + c] (r < rows, c < cols) = element (row0 + r, col0 + c) of the seeded logical
 * matrix `tensor_id` with `src_ld` columns: fp16(mean + std * N(0,1)), a pure function of
 * (seed, tensor_id, element index).  transpose = 1 writes the window transposed, dst[c*dst_ld + r];
 * transpose = 2 / 3 also transposes but sends logical column c to row (c/32)*64 + c%32 (+32 for 3),
 * the gate / value rows of the interleaved LIGER_EPI_GEGLU weight layout (cols % 32 == 0).
 */
LIGER_API int liger_fill_normal(void* dst, int rows, int cols, int dst_ld, int row0, int col0, int src_ld, uint32_t seed,
                      uint32_t tensor_id, float mean, float std, int transpose, void* stream);

/* ------------------------------------------------------------------------------------------ */
/* Dense contractions                                                                         */
/* ------------------------------------------------------------------------------------------ */

enum liger_epilogue {
  LIGER_EPI_STORE = 0,     /* C = acc (+ bias)                                                  */
  LIGER_EPI_GELU = 1,      /* C = gelu_tanh(acc + bias)                                         */
  LIGER_EPI_GEGLU = 2,     /* C[:, j] = gelu_tanh(gate_j + b) * (value_j + b); C has N/2 columns */
  LIGER_EPI_QKV_SPLIT = 3, /* acc + bias scattered to q / k / v in [B, h, S, D] layout          */
  LIGER_EPI_RESIDUAL = 4,  /* C = acc + bias + residual                                         */
  LIGER_EPI_SCATTER = 5    /* row-parallel partial sums stored straight into the owning ranks' memory */
};

/*
 * C[M, n_begin:n_end] = epilogue(A[M,K] * W[K,N]) on the tcgen05 tensor cores.
 *
 * Replaces GemmEx (src/layer/func_wrapper.h:20-27) as bound by Linear_Col / Linear_Row
 * (src/layer/linear.h:47-53, 99-105).  LIGER_EPI_QKV_SPLIT also replaces Add_QKV_bias_transpose
 * (src/layer/func_wrapper.h:57-62), LIGER_EPI_GELU replaces Add_bias_act_kernelLauncher
 * (src/layer/func_wrapper.h:90-94).
 *
 * The weight is passed pre-transposed: wt[n*ldw + k] = W[k][n] (K contiguous), which is how this
 * library stores weights (liger_fill_normal(..., transpose=1) or liger_transpose_weight produce
 * it from the reference orientation).  n_begin / n_end select a slice of output features: the
 * reference's kernel decomposition (decompose_callback, src/utils.h:218-260) maps to launches
 * with consecutive slices, and -- unlike the reference, whose slices restart at column 0 -- the
 * slices tile N exactly, so the union of the slices equals one whole launch bit for bit.
 *
 * Requirements: K % 8 == 0, lda % 8 == 0, ldw % 8 == 0, a / wt 16-byte aligned, ldc % 8 == 0 and
 * c 16-byte aligned, n_begin % 8 == 0.
 * For LIGER_EPI_GEGLU the rows of wt must be interleaved in blocks of 32 (32 gate rows, then the
 * 32 matching value rows); n_begin / n_end are in that interleaved space, multiples of 64, and
 * the result occupies columns [n_begin/2, n_end/2) of c.
 * For LIGER_EPI_QKV_SPLIT, N = 3 * heads * head_dim, row m = b * seq_len + s, and feature
 * n = which * heads * head_dim + head * head_dim + d is stored to
 * {q,k,v}_out[which][((b * heads + head) * seq_len + s) * head_dim + d].  With kv_stride > 0 the K and V
 * outputs are instead rows kv_pos + s of a KV cache laid out [B, heads, kv_stride, head_dim]
 * (prefill fills the cache from position kv_pos = 0, a decode step appends at kv_pos = kv_len).
 * For LIGER_EPI_SCATTER (the first half of a fused all-reduce: a reduce-scatter done by the GEMM's
 * own epilogue stores over NVLink, overlapped with its MMAs), row m belongs to rank
 * owner = m / ceil(M / world_size) and is stored at byte offset scatter_off of the OWNER's
 * communicator data region, laid out [world_size][ceil(M/world_size)][N], in the slot of the
 * storing rank.  liger_allreduce_fused(..., one_shot = 3) then finishes the all-reduce from the
 * local slots.  c, ldc are unused.
 * gather_comm != NULL (any epilogue; the second half of the fusion the reference's unused ReduceScatter / Allgather
 * wrappers point at, src/layer/func_wrapper.h:45-53): A is the [M, K] tensor that the most recent
 * liger_allgather_push(gather_comm, gather_channel, ...) is delivering, rank r's rows being
 * [r*ceil(M/ws), (r+1)*ceil(M/ws)).  The launch does not wait for the gather: every tile's TMA producer waits
 * (bounded, LIGER_DEV_TIMEOUT on failure) for the row blocks it is about to load, and row tiles are walked in
 * arrival order, this rank's own rows first, so the transfer runs underneath the contraction.  Issue the
 * liger_allgather_push call before this one (host order); a, lda must address the gathered tensor itself.
 */
struct liger_comm;
typedef struct liger_gemm_args {
  const void* a;        /* [M, K] fp16 */
  const void* wt;       /* [N, K] fp16 */
  void* c;              /* [M, ldc] fp16 (unused for QKV_SPLIT) */
  const void* bias;     /* [N] fp16 or NULL */
  const void* residual; /* [M, ldr] fp16, LIGER_EPI_RESIDUAL only */
  void* q_out;          /* LIGER_EPI_QKV_SPLIT only */
  void* k_out;
  void* v_out;
  int m, n, k;
  int lda, ldw, ldc, ldr;
  int n_begin, n_end;
  int epilogue;
  int seq_len, heads, head_dim; /* LIGER_EPI_QKV_SPLIT only */
  int kv_stride, kv_pos;        /* LIGER_EPI_QKV_SPLIT only: see above; 0, 0 for plain [B, h, S, D] outputs */
  struct liger_comm* scatter_comm; /* LIGER_EPI_SCATTER only */
  size_t scatter_off;              /* LIGER_EPI_SCATTER only */
  /* A is being all-gathered: see below.  NULL / 0 for an A operand that is complete. */
  struct liger_comm* gather_comm;
  int gather_channel;
} liger_gemm_args;

LIGER_API int liger_gemm_fp16(const liger_gemm_args* args, void* stream);

/* dst[n*K + k] = src[k*N + n]: imports a weight from the reference orientation W[k][n]
 * (src/layer/linear.h:40,92) into the K-contiguous layout liger_gemm_fp16 reads.  With
 * interleave32 != 0, N must be a multiple of 64 and output row block order becomes
 * (32 rows of the first half, 32 rows of the second half, ...), the LIGER_EPI_GEGLU layout. */
LIGER_API int liger_transpose_weight(const void* src, void* dst, int k, int n, int interleave32, void* stream);

/* ------------------------------------------------------------------------------------------ */
/* Attention                                                                                  */
/* ------------------------------------------------------------------------------------------ */

/*
 * out[b*S + s, head*D + d] = sum_k softmax_k(scale * q.k + (1 - mask) * -10000) v  -- one kernel for
 * the reference's QK^T batched GEMM, masked softmax, P*V batched GEMM and head-merge transpose
 * (src/layer/bert_layer.h:145-168; Attn_softmax_kernel and Transpose_kernel,
 * src/layer/func_wrapper.h:71-81).  q, k, v are [B, h, S, D] (the layout LIGER_EPI_QKV_SPLIT
 * writes); out is [B*S, ldo] with ldo >= h*D.  mask is [B, S, S] fp16 of 0/1 shared over heads
 * (src/cuda/attention_kernels.cu:544), or NULL with causal = 1 for a causal mask or causal = 0
 * for none.  Scores never leave the chip; the softmax is computed in fp32 (the reference's half
 * path scales, masks and exponentiates in fp16: src/cuda/attention_kernels.cu:561-567).
 * D must be 64 or 128; S is unrestricted (the reference stops at 2048).
 */
LIGER_API int liger_attention_prefill(const void* q, const void* k, const void* v, const void* mask, void* out, int batch,
                            int heads, int seq_len, int head_dim, int ldo, float scale, int causal, void* stream);

/*
 * Decode step: one new query token per sequence against a KV cache.  q is [B, h, D];
 * k_cache / v_cache are [B, h, L_max, D] holding kv_len valid positions; out is [B, ldo].
 * The KV range is split across CTAs; partial results live in `scratch` (float,
 * liger_attention_decode_scratch_bytes() bytes).  No reference counterpart: the reference has no
 * KV cache or decode path.
 */
LIGER_API size_t liger_attention_decode_scratch_bytes(int batch, int heads, int head_dim, int kv_len);
LIGER_API int liger_attention_decode(const void* q, const void* k_cache, const void* v_cache, void* out, void* scratch,
                           int batch, int heads, int kv_len, int kv_stride, int head_dim, int ldo, float scale,
                           void* stream);

/*
 * liger_attention_decode for callers that cannot allocate device memory.  No counterpart in the
 * reference (it has no decode path at all); it exists for hosts where cudaMalloc is off limits at
 * the call site -- a serving loop whose memory pool is sized and frozen at start-up, a plugin that
 * runs inside someone else's allocator, code between two points where device allocation would
 * synchronise the device or is simply forbidden by policy.  The split-KV partials go to a 16 MiB
 * buffer built into the library image (one per GPU that loads the library, held until the
 * process exits) instead of caller scratch; the call itself performs no cudaMalloc / cudaFree and
 * calls nothing that allocates.  q, k_cache, v_cache and out are still the caller's.
 *
 * Limits and rules:
 *  - batch * heads * ceil(kv_len / 256) * (head_dim + 2) * 4 bytes must not exceed
 *    liger_attention_decode_noalloc_max_bytes() (16 MiB); larger requests return
 *    LIGER_ERR_TOO_LARGE and launch nothing (use liger_attention_decode with your own scratch).
 *  - The first call on each device looks up the device address of the built-in buffer
 *    (cudaGetSymbolAddress); make that first call outside any stream capture.
 *  - All calls on a device share the one buffer and it keeps whatever the last call left there.
 *    Each call overwrites every partial it later reads, so stale contents are never consumed, but
 *    two calls that overlap on the GPU (different streams, no ordering between them) race on the
 *    buffer: serialise them.
 */
LIGER_API size_t liger_attention_decode_noalloc_max_bytes(void);
LIGER_API int liger_attention_decode_noalloc(const void* q, const void* k_cache, const void* v_cache, void* out, int batch,
                                             int heads, int kv_len, int kv_stride, int head_dim, int ldo, float scale,
                                             void* stream);

/* ------------------------------------------------------------------------------------------ */
/* Row-wise operators                                                                         */
/* ------------------------------------------------------------------------------------------ */

/* y = LayerNorm(x) over the last dimension, eps 1e-6, biased variance, fp32 statistics.
 * Replaces Layer_Norm (src/layer/func_wrapper.h:110-114 -> src/cuda/cuda_kernels.cu:463-532). */
LIGER_API int liger_layernorm(const void* x, const void* gamma, const void* beta, void* y, int m, int n, void* stream);

/* out = in + out + bias (stored in place), norm = LayerNorm(out) when norm != NULL.
 * Replaces Add_bias_input_layernorm_2_kernelLauncher and Add_bias_input_kernelLauncher
 * (src/layer/func_wrapper.h:96-108 -> src/cuda/cuda_kernels.cu:360-461). bias may be NULL. */
LIGER_API int liger_add_bias_input_layernorm(const void* in, const void* gamma, const void* beta, const void* bias, void* out,
                                   void* norm, int m, int n, void* stream);

/* x = gelu_tanh(x + bias) in place. Replaces Add_bias_act_kernelLauncher
 * (src/layer/func_wrapper.h:90-94 -> src/cuda/cuda_kernels.cu:71-84,302-319). */
LIGER_API int liger_add_bias_gelu(void* x, const void* bias, int m, int n, void* stream);

/* {q,k,v}_out[b][h][s][d] = {Q,K,V}[b*S+s][h*D+d] + bias. Replaces Add_QKV_bias_transpose
 * (src/layer/func_wrapper.h:57-62 -> src/cuda/attention_kernels.cu:133-163,226-329). */
LIGER_API int liger_add_qkv_bias_transpose(void* q_out, void* k_out, void* v_out, const void* q, const void* bq, const void* k,
                                 const void* bk, const void* v, const void* bv, int batch, int seq_len, int heads,
                                 int head_dim, void* stream);

/* dst[b*S+s][h*D+d] = src[b][h][s][d]. Replaces Transpose_kernel
 * (src/layer/func_wrapper.h:77-81 -> src/cuda/attention_kernels.cu:693-742). */
LIGER_API int liger_transpose_heads(void* dst, const void* src, int batch, int seq_len, int heads, int head_dim, void* stream);

/* ------------------------------------------------------------------------------------------ */
/* Tensor-parallel communication over NVLink / NVSwitch peer memory                           */
/* ------------------------------------------------------------------------------------------ */

/*
 * A communicator owns one "symmetric segment" per rank: a device buffer of the same size on every
 * GPU that every peer maps, so kernels address peer memory directly by (rank, offset).  It
 * replaces the reference's NCCL communicator (createNcclComm, src/communicator.h:9-41: the
 * ncclUniqueId broadcast becomes an exchange of LIGER_COMM_HANDLE_BYTES-byte handles over
 * whatever the host already uses -- MPI_Bcast / all-gather, a torch.distributed group ...).
 *
 *   liger_comm_create   allocate the local segment (data_bytes + flag words), one process per GPU
 *   liger_comm_export   write this rank's handle
 *   liger_comm_connect  given all ranks' handles (rank order), map every peer's segment
 *
 * Ranks that live in one process (several GPUs driven by one host thread each) are detected by
 * process id and mapped with peer access instead of IPC handles.  world_size <= 8.
 * `channels` independent flag sets let collectives of different in-flight requests proceed
 * without sharing barrier state; all ranks must launch the collectives of one channel in the
 * same order.
 */
typedef struct liger_comm liger_comm;
#define LIGER_COMM_HANDLE_BYTES 128
#define LIGER_COMM_MAX_RANKS 8

LIGER_API int liger_comm_create(liger_comm** out, int rank, int world_size, size_t data_bytes, int channels);
LIGER_API int liger_comm_export(liger_comm* comm, void* handle_out);
LIGER_API int liger_comm_connect(liger_comm* comm, const void* all_handles);
LIGER_API int liger_comm_destroy(liger_comm* comm);
/* Base address of this rank's data region (offsets below are bytes from this base). */
LIGER_API void* liger_comm_data(liger_comm* comm);
LIGER_API size_t liger_comm_data_bytes(liger_comm* comm);
LIGER_API int liger_comm_rank(liger_comm* comm);
LIGER_API int liger_comm_world_size(liger_comm* comm);
LIGER_API int liger_comm_channels(liger_comm* comm);

/*
 * Where the fused all-reduce launches of `channel` spent their time since the last reset, summed over
 * launches, in microseconds: out_us[0] waiting for peers at the entry barrier (skew between ranks),
 * out_us[1] reducing / normalising / storing, out_us[2] waiting at the exit barrier; out_us[3] = number
 * of launches.  Synchronises the device copy; call it outside timed regions.
 */
LIGER_API int liger_comm_timing(liger_comm* comm, int channel, int reset, double out_us[4]);

/*
 * Which of the two few-row kernels (M <= 32) liger_gemm_fp16 takes for an [n, k] weight on a GPU with sm_count SMs,
 * without launching anything (no GPU needed): out[0] = 2 cluster kernel / 3 stream-K kernel, out[1] = CTAs per
 * cluster (K splits; 1 for stream-K), out[2] = 64-deep k-blocks each CTA streams, out[3] = CTAs of the launch.
 * The choice depends on the whole weight only, never on the slice [n_begin, n_end) being computed.  The reference
 * has no counterpart (one cuBLAS heuristic call per GEMM, src/layer/func_wrapper.h:20-27).
 */
LIGER_API int liger_gemm_smallm_plan(int n, int k, int sm_count, int out[4]);

/*
 * All-reduce (sum over ranks) of the row-parallel partials, fused with what follows it in the layer.
 * Replaces Allreduce (src/layer/func_wrapper.h:40-43, bound at src/layer/linear.h:55-60) together
 * with the residual / LayerNorm kernel after it (Layer_Norm, src/layer/func_wrapper.h:110-114, or
 * add_bias_input_layernorm_2, src/cuda/cuda_kernels.cu:360-409).
 *
 * Every rank holds its partial [M, N] fp16 at byte offset partial_off of its segment.  Rank r owns
 * rows [r*ceil(M/ws), (r+1)*ceil(M/ws)).  For each owned row in [row_begin, row_end):
 *     t = sum_p partial_p[row]            fp32; order: p = row mod ws first, then increasing rank, cyclic
 *     if hidden:  t += residual_in[row] + bias ; hidden[row] = fp16(t)   (residual stream, local, owner
 *                 rows; residual_in may equal hidden, or be NULL to mean hidden)
 *     if gamma:   o = LayerNorm(fp16(t)) * gamma + beta   else   o = fp16(t)
 *     store o to row `row` of the [M, N] tensor at byte offset out_off of EVERY rank's segment
 * preceded and followed by a cross-rank barrier on flag set `channel`, so that a kernel launched
 * after this one on the same stream sees all rows.  With one_shot != 0 every rank instead reduces
 * all rows itself and stores only locally (latency-bound sizes; hidden is then updated for all
 * rows on every rank).  one_shot == 3: two-shot, but the partials were already scattered to their
 * owners by GEMMs with LIGER_EPI_SCATTER (partial_off is then the [world_size][rows][N] receive
 * region) and the reduction reads local memory only.  one_shot == 2 turns the call into an all-gather: each rank's own rows of its
 * partial are taken as they are (no sum over peers) and stored to every rank.
 * one_shot == 5: input as for 3, but the finished rows are stored into this rank's own segment only and there is no
 * exit barrier -- the first half of a split collective whose second half is liger_allgather_ce on another stream.
 * one_shot == 6: as 1, without the exit barrier.  Safe only if consecutive calls on the channel read their partials
 * from two alternating buffers: the entry barrier of call k+1 then tells every rank that all ranks have finished
 * reading the input of call k, before anything rewrites it for call k+2 (a decode step's two all-reduces per layer).
 * Waits on peers are bounded; on timeout the device status word is set.
 * N % 8 == 0, N <= 16384.  row_begin / row_end allow the collective to be issued in slices
 * (decompose_comm_callback, src/utils.h:262-281).
 */
LIGER_API int liger_allreduce_fused(liger_comm* comm, int channel, size_t partial_off, size_t out_off,
                                    const void* residual_in, void* hidden, const void* bias, const void* gamma,
                                    const void* beta, int m, int n, int row_begin, int row_end, int one_shot,
                                    void* stream);

/*
 * The same collective (two-shot, rows [row_begin, row_end)) with all inter-GPU data movement on the
 * copy engines instead of SM loads / stores: peer copies deliver every rank's slice of the partials
 * (plain [M, N] layout at partial_off) into the owners' receive slots ([world_size][rows][N] at
 * recv_off), a small kernel reduces the owned rows from local memory (+ residual + LayerNorm) into
 * the local [M, N] tensor at out_off, and peer copies distribute the finished rows; one-warp barrier
 * kernels order the phases across ranks.  Meant for interleaved execution: the SMs stay free for the
 * GEMMs of the other requests (or micro-batches) that run under the transfer.  Same arithmetic and
 * summation order as liger_allreduce_fused.
 */
LIGER_API int liger_allreduce_ce(liger_comm* comm, int channel, size_t partial_off, size_t recv_off, size_t out_off,
                                 const void* residual_in, void* hidden, const void* bias, const void* gamma,
                                 const void* beta, int m, int n, int row_begin, int row_end, void* stream);

/*
 * All-gather by the copy engines, the second half of a split all-reduce (the reference's unused Allgather
 * wrapper, src/layer/func_wrapper.h:50-53, is the nearest counterpart): rows [row_begin, row_end) that this
 * rank owns (rank r owns rows [r*ceil(m/ws), (r+1)*ceil(m/ws)) of the [m, n] tensor at out_off) are copied to
 * the same place in every peer's segment with one peer copy per peer, followed by a one-warp barrier kernel on
 * `channel`, after which every rank holds all rows.  No SM moves data, so the transfer runs underneath the
 * kernels of another stream.  Use a channel of its own when other collectives are in flight on other streams.
 */
LIGER_API int liger_allgather_ce(liger_comm* comm, int channel, size_t out_off, int m, int n, int row_begin, int row_end,
                                 void* stream);

/*
 * All-gather whose consumer is the next GEMM.  Rank r's rows of the [m, n] tensor at out_off go to every peer's
 * segment, in row blocks of 256 rows, peer by peer (rank-1, rank-2, ...); each delivered (row block, peer) is
 * announced in the peer's flag line of `ready_channel`.  The data is moved by the copy engines (one peer copy per
 * row block and peer, followed by a 4-byte copy that publishes the flag), so no SM is taken from the GEMM that
 * runs beside the transfer.  A GEMM launched with
 * liger_gemm_args.gather_comm / gather_channel = (comm, ready_channel) starts before the gather has finished and
 * waits per tile.  A one-warp barrier kernel on `barrier_channel` follows the push, so that anything ordered
 * after this call on `stream` sees all rows.  Both channels must be used for nothing else while other
 * collectives are in flight on other streams.  (Nearest reference counterpart: the unused Allgather wrapper,
 * src/layer/func_wrapper.h:50-53.)
 */
LIGER_API int liger_allgather_push(liger_comm* comm, int ready_channel, int barrier_channel, size_t out_off, int m, int n,
                                   void* stream);

/* ------------------------------------------------------------------------------------------ */
/* The layer stack and the serving entry points                                               */
/* ------------------------------------------------------------------------------------------ */

/*
 * Configuration: the reference's eight integers (src/main.cu:14-21; BertInitParam,
 * src/context.h:58-85) followed by the settings the reference hard-codes or lacks.
 * liger_model_config_init() fills in the reference's defaults.
 */
typedef struct liger_model_config {
  int max_batch_size, max_seq_len, head_num, size_per_head, layer_num, kernel_num, factor;
  int rq_interval;   /* microseconds between requests = 1e6 / arrival rate (src/main.cu:33) */
  int graph;         /* 0: reference graph (post-LayerNorm, no residual); 1: pre-LayerNorm + residual */
  int act;           /* 0: bias + GELU; 1: GeGLU */
  int ffn_inner;     /* 0 -> 4 * hidden */
  int causal;        /* 1: causal mask by construction; 0: mask tensor (all ones unless set) */
  uint32_t seed;
  int num_requests;  /* 150 (src/schedule.h:295) */
  int ignore_num;    /* 20 (src/schedule.h:327) */
  int schedule_deep; /* 6 (src/schedule.h:30) */
  float contention;  /* 0.8 (src/schedule.h:249); 0: the per-direction factors measured by the profile run */
  int poisson;       /* 0: fixed-interval arrivals, 1: exponential gaps */
  int min_seq_len;   /* 16 */
  int seq_round;     /* request lengths are rounded up to a multiple of this (profile bucket) */
  int workspace_slots;
  int kv_capacity;
  float min_slice_efficiency; /* 0 (reference: any GEMM slice that fits the window, src/init.h:226-259); e.g. 0.7: only
                                 slices profiled at >= 70 % of the whole kernel's rate */
} liger_model_config;

LIGER_API void liger_model_config_init(liger_model_config* cfg);

typedef struct liger_model liger_model;

/* Bytes of communicator data region a model with this configuration needs (0 for world_size 1). */
LIGER_API size_t liger_model_comm_bytes(const liger_model_config* cfg, int world_size);

/*
 * Builds the layer stack on the current device: seeded weights (each rank keeps its tensor-parallel
 * shard of the full-shape tensors), per-request workspaces, and the function-assembly machinery.
 * Replaces `new Bert_Model<T>(BertParams, SParams, k, n, workspace)` (src/layer/bert.h:88-102,
 * src/test_schedule.h:35).  comm may be NULL when world_size == 1.
 */
LIGER_API int liger_model_create(liger_model** out, const liger_model_config* cfg, int rank, int world_size,
                                 liger_comm* comm);
LIGER_API int liger_model_destroy(liger_model* model);

/*
 * One forward pass: assembles the kernel vector of a (batch, seq_len) request
 * (Bert_Model::forward, src/layer/bert.h:104-115) and launches every kernel in order on `stream`
 * (what Scheduler::run_sequential does for one request, src/schedule.h:204-219).  input / output are
 * [batch*seq_len, hidden] fp16 in device memory.  slot selects the activation workspace (-1: round
 * robin).  Returns the number of kernels launched, or a negative error.
 */
LIGER_API int liger_model_forward(liger_model* model, const void* input, void* output, int batch, int seq_len, int slot,
                                  void* stream);
/*
 * One decode step: `batch` sequences, one new token each (input / output [batch, hidden]), against
 * the model's KV caches holding kv_len positions (cfg.kv_capacity > kv_len; pre-LayerNorm graph).
 * Per layer the token's K and V are appended at position kv_len by the QKV GEMM's epilogue and a
 * split-KV attention kernel streams the cache once.  liger_model_fill_kv_cache() loads the caches
 * with seeded N(0,1) values (tensor ids 0x10001 + 2*layer / 0x10002 + 2*layer, logical layout
 * [batch][heads][kv_capacity][head_dim]).  The reference has no decode path or KV cache; these two
 * entry points exist for the decode configuration of the benchmark suite.  Returns the number of
 * kernels launched.
 */
LIGER_API int liger_model_decode(liger_model* model, const void* input, void* output, int batch, int kv_len, int slot,
                                 void* stream);
LIGER_API int liger_model_fill_kv_cache(liger_model* model);

/*
 * Interleaving inside one request.  With micro_batches = n > 1 and world_size > 1, a forward pass
 * whose batch divides by n is split into n micro-requests (consecutive groups of sequences) that
 * run on n internal streams and n consecutive workspace slots starting at `slot`, launched
 * segment by segment in turn, so that the all-reduces of one micro-request overlap the GEMMs of
 * the others; the caller's stream waits for all of them.  This is the reference scheduler's
 * interleaving of one request's communication with other requests' computation
 * (Scheduler::run_stream_sync, src/schedule.h:221-278) applied to the halves of a single batch.
 * Results are identical to the un-split pass (rows are independent across sequences).
 */
LIGER_API int liger_model_set_micro_batches(liger_model* model, int micro_batches);
/*
 * How the micro-requests of liger_model_set_micro_batches share the GPU.
 *   1 (default): one compute stream runs the compute segments of all micro-requests in turn; every all-reduce is
 *      split into the reduce-scatter done by the row-parallel GEMM's epilogue, a short local reduction
 *      (+ residual + LayerNorm) on the compute stream, and an all-gather by the copy engines on a second stream
 *      (liger_allgather_ce) that runs underneath the other micro-request's next compute segment.  Needs a
 *      communicator with at least 2 * workspace_slots channels; with fewer, mode 0 is used.
 *   0: one stream per micro-request, all-reduces entirely in kernels (liger_allreduce_fused).
 *   2: no micro-requests at all: the whole batch on the caller's stream; after the local reduction the all-gather
 *      (liger_allgather_push, a copy kernel small enough to share the SMs with a GEMM) runs on a second stream
 *      beside the column-parallel GEMM that consumes it, which starts at once and waits tile by tile for its rows
 *      (liger_gemm_args.gather_comm).  Needs 3 * workspace_slots channels; with fewer, the modes above apply.
 * All give the bits of the un-split pass.  This is the reference's decomposition + two-stream interleaving
 * (src/init.h:226-259, src/schedule.h:221-278) re-derived for a GPU whose persistent GEMMs leave no SM resources
 * for a concurrent communication kernel: the decomposition is along the batch, and the overlapped half of the
 * communication uses no SM.
 */
LIGER_API int liger_model_set_overlap(liger_model* model, int mode);
/*
 * After liger_model_kernel_times() on passes run with mode 1: out[0] = milliseconds the compute stream spent
 * blocked waiting for an all-gather (exposed communication beyond the local reductions, which are counted under
 * kernel names 3 and 6), out[1] = number of such waits, out[2] = milliseconds of the copy-engine all-gathers on the
 * communication stream, out[3] = their number.  Clears the sums.
 */
LIGER_API int liger_model_overlap_times(liger_model* model, double out[4]);

/* world_size > 1, liger_model_forward_host only.  sharded = 1: every rank copies rows
 * [rank * ceil(M / world_size), ...) of the result -- the rows it uploaded -- to the same offsets of ITS
 * host_output, so that ranks whose host_output is one shared, pinned host buffer fill it together and each
 * PCIe link carries 1/world_size of the result.  sharded = 0 (default): rank 0 downloads everything.
 * (No counterpart in the reference.) */
LIGER_API int liger_model_set_output_sharding(liger_model* model, int sharded);

/* Diagnostics for interleaved passes: with enable != 0 the next interleaved pass records an event
 * before and after every kernel on its own stream; a later call returns, for the last such pass,
 * kernel name, stream index and the enqueue-order event times in ms since the pass started (up to
 * `capacity` entries; returns the count).  Event times bound a kernel's execution from above: a
 * kernel may wait between its "before" event and its actual start. */
LIGER_API int liger_model_timeline(liger_model* model, int enable, int capacity, int* names, int* streams,
                                   double* start_ms, double* end_ms);

/* Same with HOST buffers, all on `stream`; returns after enqueueing (synchronise the stream before
 * reading host_output).  world_size == 1: the whole input is copied to the device and the whole
 * result back.  world_size > 1: every rank passes the same full host input but uploads only its
 * own 1/world_size of the rows, which an all-gather over peer memory completes on every GPU; the
 * result is copied to host_output on rank 0 only (other ranks leave host_output untouched), unless
 * liger_model_set_output_sharding() asked for every rank to download its own rows.
 * (No counterpart in the reference, whose buffers never leave the device: src/test_schedule.h:19-47.) */
LIGER_API int liger_model_forward_host(liger_model* model, const void* host_input, void* host_output, int batch,
                                       int seq_len, int slot, void* stream);
/*
 * Per-kernel timing of liger_model_forward[_host]: when enabled, the pass records a CUDA event on
 * `stream` before and after every kernel it launches.  liger_model_kernel_times() waits for the
 * recorded events, adds the elapsed milliseconds and launch counts per kernel name (0..8, see
 * liger_model_forward) into ms[9] / launches[9], and clears the record.  This is the measurement
 * Scheduler::profile makes one kernel at a time (src/schedule.h:93-112), taken in situ.
 */
LIGER_API int liger_model_set_kernel_timing(liger_model* model, int enable);
LIGER_API int liger_model_kernel_times(liger_model* model, double ms[9], long long launches[9]);
/* Algorithmic FLOPs of kernel `name` (GEMMs: 2*M*N*K of this rank's shard; attention: QK^T + PV,
 * halved when causal) and the bytes it must move (operands + results once), for one request of
 * (batch, seq_len); 0 for names that do not exist in this configuration. */
LIGER_API int liger_model_kernel_work(liger_model* model, int name, int batch, int seq_len, double* flops,
                                      double* bytes);
/* Attention mask [max_batch, S, S] fp16 of 0/1 used when cfg.causal == 0 (NULL: all ones). */
LIGER_API int liger_model_set_mask(liger_model* model, const void* mask);

/* Cross-rank callbacks the serving loop needs: broadcast one int from rank 0, and a barrier.  Both
 * may be NULL when world_size == 1. */
typedef int (*liger_bcast_int_fn)(void* ctx, int* value);
typedef int (*liger_barrier_fn)(void* ctx);

typedef struct liger_serving_metrics {
  int records;                  /* requests counted (after dropping the first ignore_num) */
  int launch_errors;
  double total_duration_ms;     /* the reference's Total_Duration */
  double throughput_samples_s;  /* the reference's Throughput */
  double average_latency_ms;    /* the reference's Average Latency */
  double tokens_per_s, p50_latency_ms, p99_latency_ms, mean_gpu_ms;
  long long tokens;
  long long segments, secondary_launches, decompositions;
} liger_serving_metrics;

#define LIGER_MODE_PROFILE 0     /* test_profile     (src/test_schedule.h:80-104) */
#define LIGER_MODE_SCHEDULE 1    /* test_schedule    (src/test_schedule.h:19-47): Liger's interleaved schedule */
#define LIGER_MODE_NO_SCHEDULE 2 /* test_no_schedule (src/test_schedule.h:50-78): unscheduled baseline */

/*
 * Runs one of the three entry points on an existing model.  Profile files are read / written in
 * `profile_dir` under the reference's names Main_<ws>_<size_per_head>_<head_num>_<max_batch>_<max_seq>.json
 * and Sub_... (rank 0 writes, every rank reads).  metrics may be NULL (and is unused for PROFILE).
 */
LIGER_API int liger_serve(liger_model* model, int mode, liger_bcast_int_fn bcast, liger_barrier_fn barrier, void* ctx,
                          const char* profile_dir, int print, liger_serving_metrics* metrics);

/*
 * Profile files (the scheduler's cost model; format of MainDictToFile / SubDictToFile,
 * src/utils.h:106-215).  liger_profile_rewrite() parses `in_path` (is_sub = 0: scalar durations,
 * 1: arrays of factor-1 durations) and writes it back through the library's writer; entries and
 * the sum of all durations are returned.  Malformed input (the reference's reader throws) gives
 * LIGER_ERR_INVALID with the parse position in liger_last_error().  out_path may be NULL.
 */
LIGER_API int liger_profile_rewrite(const char* in_path, const char* out_path, int is_sub, int* entries, double* duration_sum);
/*
 * What the scheduler's cost model predicts for kernel `name` of a (batch, seq_len) request, from the Main profile at
 * main_path taken for a model of (max_batch, max_seq): the profiled value where there is one; otherwise linear
 * interpolation between the nearest profiled lengths of the same batch size, extrapolation in proportion to the length
 * beyond the last one, and the nearest profiled batch size scaled by the token count.  The reference looks the exact
 * key up and uses 0 for everything else (src/schedule.h:166), hence its profile over every integer length
 * (src/test_schedule.h:103).
 */
LIGER_API int liger_profile_predict(const char* main_path, int max_batch, int max_seq, int name, int batch, int seq_len,
                                    double* duration_ms);

/*
 * The scheduling logic on a simulated device (no GPU): a layer is given as kernels_per_layer
 * (type, milliseconds at max_batch*max_seq tokens) pairs, durations scale with the token count, a
 * GEMM slice of n/factor costs slice_overhead_ms + n/factor of the whole, and two kernels running
 * at once each progress at overlap_rate.  Runs `mode` (SCHEDULE or NO_SCHEDULE) over the seeded
 * request schedule and reports every launch.  Used by the CPU tests of the scheduler.
 */
typedef struct liger_sim_kernel { int type; float duration_ms; } liger_sim_kernel; /* type: 0 COMM, 1 COMP, 2 GEMM */
typedef struct liger_sim_launch {
  int request, layer, name, stream, units_begin, units_end;
  float duration_ms;
  double t_start_ms, t_end_ms;
} liger_sim_launch;
LIGER_API int liger_sim_serve(const liger_model_config* cfg, const liger_sim_kernel* layer_kernels,
                              int kernels_per_layer, int mode, double overlap_rate, double slice_overhead_ms,
                              liger_sim_launch* log, int log_capacity, int* log_count,
                              liger_serving_metrics* metrics);
/* The same as one rank of `world_size`: admissions are decided by rank 0 and received through
 * `bcast` (as in liger_serve); this rank's host clock runs `host_skew_ms` ahead, and its device is
 * `device_slowdown` times slower, so that ranks would admit at different moments if they decided
 * on their own. */
LIGER_API int liger_sim_serve_rank(const liger_model_config* cfg, const liger_sim_kernel* layer_kernels,
                                   int kernels_per_layer, int mode, double overlap_rate, double slice_overhead_ms,
                                   int rank, int world_size, liger_bcast_int_fn bcast, liger_barrier_fn barrier, void* ctx,
                                   double host_skew_ms, double device_slowdown, liger_sim_launch* log, int log_capacity,
                                   int* log_count, liger_serving_metrics* metrics);

#ifdef __cplusplus
}
#endif
#endif /* LIGER_B200_H */

/* libfdk_b200 -- C ABI of the B200 (sm_100a) fused-dequantisation kernels.
 *
 * Drop-in boundary for the LUT hot path of graphcore-research/
 * fused-dequantisation-kernels ("fdk").  The reference reaches its kernels
 * through Python operator functions that take torch tensors, write into a
 * caller-allocated `out` and launch on the current CUDA stream
 * (src/fdk/kernels.py:158-182 run_mv_lut, :460-489 run_mm_lut); its one native
 * extension shows the C convention it uses for compiled code:
 * `int marlin_cuda(const void* A, const void* B, void* C, void* s, ...,
 * cudaStream_t stream, ...)` returning 0 or a small error code that the
 * binding turns into an exception (src/fdk/marlin/marlin_cuda.cpp:25-45,
 * 63-66, 84-93).  This header follows that convention: plain pointers and
 * sizes, an explicit stream, an int status, no torch types.
 *
 * Every pointer is a DEVICE pointer unless the parameter name ends in
 * `_host`.  `stream` is a cudaStream_t passed as void* (NULL = legacy default
 * stream).  All calls are asynchronous on `stream`, never synchronise, and,
 * except where a comment says otherwise, allocate nothing, so they can be
 * captured in a CUDA graph as the reference's timing harness does
 * (src/fdk/bench.py:67-99, src/fdk/models.py:329-331).
 *
 * 16-bit floating-point data is bfloat16 (FDK_DTYPE_BF16) or IEEE half
 * (FDK_DTYPE_F16); the reference uses bf16 for its LUT kernels and fp16 for
 * its Marlin selectors (src/fdk/models.py:486-491).
 */
#ifndef FDK_B200_H_
#define FDK_B200_H_

#include <stddef.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

/* ---- status codes (0 = success, like marlin_cuda's return value) ---------- */
#define FDK_OK 0
#define FDK_ERR_BAD_ARG 1   /* null pointer, non-positive size, unknown dtype/flag      */
#define FDK_ERR_SHAPE 2     /* shape the kernels do not take (cf. ERR_PROB_SHAPE,
                               src/fdk/marlin/marlin_cuda.cpp:25): bits not in
                               {1,2,3,4,8}, k or block_size not a multiple of 64 ...   */
#define FDK_ERR_ALIGN 3     /* pointer not 16-byte aligned where the kernels need it    */
#define FDK_ERR_ARCH 4      /* current device is not compute capability 10.x            */
#define FDK_ERR_CUDA 5      /* a CUDA runtime call failed; see fdk_last_error_detail()  */
#define FDK_ERR_WORKSPACE 6 /* workspace missing or smaller than fdk_workspace_size()   */

#define FDK_DTYPE_BF16 0
#define FDK_DTYPE_F16 1

/* flags of fdk_linear_lut */
#define FDK_FLAG_PDL 1u /* launch with programmatic stream serialisation: the kernel's
                           weight prefetch may overlap the tail of the previous kernel
                           on the stream; x / out / workspace are only touched after
                           the previous kernel has completed.                          */
#define FDK_FLAG_SILU_PAIRS 2u /* the weight rows come in groups of 64: 32 "gate" rows, then
                           the 32 matching "up" rows; the kernel writes
                           out[m, n / 2] = silu(gate) * up instead of the [m, n] products,
                           with the roundings of fdk_linear_lut (as it is up to 16 rows)
                           followed by fdk_silu_mul (group 32).  m <= 16, n a multiple
                           of 64.                                                      */

#define FDK_FLAG_NO_SYNC 4u   /* fdk_linear_lut_host only: return without synchronising the
                           stream; out_host is valid once the caller has synchronised it,
                           and x_host must stay untouched until then.  Calls on one stream
                           may follow each other (they share the staging buffers in stream
                           order), so that copies and kernels of successive calls overlap
                           the host's work.                                             */

/* Library version: major*10000 + minor*100 + patch. */
int fdk_version(void);

/* Static text for a status code. */
const char* fdk_status_string(int status);

/* Detail of the last non-zero status returned on the calling thread
 * (e.g. which argument, or the CUDA error string).  Never NULL. */
const char* fdk_last_error_detail(void);

/* Size in bytes of the tiled buffer for an [n, k] matrix of `bits`-bit codes.
 * Host-only arithmetic.  Replaces nothing in the reference: the tiled layout
 * is this library's own (the reference's kernels read the packed tensors of
 * src/fdk/models.py:94-104 directly). */
int fdk_tiled_size(int n, int k, int bits, size_t* bytes_host);

/* Offline repacker: the reference's packed tensors -> tiled buffer.
 *   codes  [n, k*bits/8] uint8, element 0 of a byte in the high bits
 *          (src/fdk/models.py:94-102); for bits == 3, which the reference
 *          does not have, one MSB-first bit stream per row.
 *   scale  [n, k/block_size] 16-bit floats (src/fdk/models.py:81-88).
 * block_size must be a multiple of 64 and divide k; k a multiple of 64.
 * `tiled` must hold fdk_tiled_size() bytes and be 16-byte aligned.
 * Stands where QuantisedLinear.create hands its tensors to the module
 * (src/fdk/models.py:104). */
int fdk_repack(const void* codes, const void* scale, int n, int k, int bits, int block_size,
               void* tiled, void* stream);

/* Inverse of fdk_repack (tests, state_dict export).  block_size as above; the
 * scale written for a block_size > 64 is that of the first 64-run. */
int fdk_unpack(const void* tiled, int n, int k, int bits, int block_size, void* codes, void* scale,
               void* stream);

/* Bit-exact dequantisation, W[n,k] = dtype(float(lut[byte][j]) * float(scale[n, k/block_size])),
 * i.e. the first two lines of mm_lut_ref (src/fdk/kernels.py:23-24).
 *   lut    [256, 8/bits] byte table (src/fdk/models.py:103); for bits == 3 the
 *          plain 8-entry codebook.
 *   w_out  [n, k] 16-bit floats, 16-byte aligned. */
int fdk_dequantise(const void* codes, const void* lut, const void* scale, int n, int k, int bits,
                   int block_size, int dtype, void* w_out, void* stream);

/* Same result, read from the tiled buffer. */
int fdk_dequantise_tiled(const void* tiled, const void* lut, int n, int k, int bits, int dtype,
                         void* w_out, void* stream);

/* Scratch needed by fdk_linear_lut on the current device (partial sums of row tiles
 * whose K range is split over several SMs, and their use counts).  One workspace per stream that runs the kernels
 * concurrently.  Compare Marlin's `workspace` (src/fdk/marlin/__init__.py:37-51,
 * marlin_cuda.cpp:65-66): caller-allocated, zeroed once (fdk_workspace_init), reusable
 * by every later call on the same stream without clearing. */
int fdk_workspace_size(size_t* bytes_host);

/* Zeroes the workspace (cudaMemsetAsync).  Call once after
 * allocating.  The first call on a device also asks the device where kernels see their
 * dynamic shared memory (one tiny kernel, synchronous), so make it outside any stream
 * capture. */
int fdk_workspace_init(void* workspace, size_t workspace_bytes, void* stream);

/* Reads the workspace's device-side status word (synchronous copy): 0 when every
 * fdk_linear_lut that used the workspace ran normally; bit 0 = a bounded wait (for another
 * CTA's partial sums, or on a copy barrier of the tensor-core kernel) ran out, bit 1 = the
 * shared-memory layout planned by the host did not match the device.  The kernels never trap or spin without limit; this is where they report.
 * No counterpart in the reference (its kernels have no device-side error reporting,
 * cf. the soft handling in src/fdk/bench.py:457-458). */
int fdk_workspace_status(const void* workspace, int* status_host);

/* Fused dequantise + matrix product, out[m, n] = x[m, k] . W[n, k]^T with W as
 * fdk_dequantise defines it but never materialised; fp32 accumulation, block
 * scale applied to the fp32 block sum.  Replaces run_mv_lut (m == 1,
 * src/fdk/kernels.py:158-182) and run_mm_lut (m > 1, src/fdk/kernels.py:460-489).
 *   x         [m, k] row-major, 16-byte aligned rows (k % 8 == 0)
 *   lut       byte table in device memory ([256, 8/bits], or the 8-entry codebook
 *             for bits == 3); may be NULL when lut_host is given
 *   lut_host  optional HOST copy of the same table.  When given it is passed to the
 *             kernel by value with the launch parameters, which saves the kernel a
 *             memory round trip before it can start (the table is 16 B .. 4 KB)
 *   out       [m, n] row-major
 *   m         >= 1, any m: up to 16 rows run the GEMV kernel (one n-tile of the tensor-core
 *             instruction up to 8 rows, two from 9), more the tcgen05 kernel.
 * Deterministic: the same inputs give the same bits on every call. */
int fdk_linear_lut(const void* x, const void* tiled, const void* lut, const void* lut_host, void* out,
                   int m, int n, int k, int bits, int dtype, void* workspace, size_t workspace_bytes,
                   unsigned flags, void* stream);

/* ---- glue of the decode step around the quantised projections ------------------------
 * The reference takes this arithmetic from transformers' LlamaForCausalLM, called from
 * Generator.step (src/fdk/models.py:245-255); these three kernels replace about ten
 * framework launches per layer.  bf16 only. */

/* Residual add fused with RMSNorm: if delta != NULL, h[rows, width] += delta (bf16 add, in
 * place); then out = weight * bf16(h * rsqrt(mean(h^2) + eps)) computed in fp32. */
int fdk_rmsnorm(void* h, const void* delta, const void* weight, void* out, int rows, int width,
                float eps, void* stream);

/* Rotary embedding fused with the KV-cache append.  qkv [rows, (q_heads + 2 kv_heads) * 128] is
 * the output of the fused q|k|v projection; *pos (device int64) is the token position.  q is
 * rotated into q_out [rows, q_heads * 128]; k is rotated and v copied into k_cache / v_cache
 * [rows, kv_heads, max_len, 128] at position *pos.  Rotate-half convention, cos/sin rounded to
 * bf16 as the framework model does.  head_dim must be 128. */
int fdk_rope_append(const void* qkv, const void* pos, void* q_out, void* k_cache, void* v_cache,
                    int rows, int q_heads, int kv_heads, int head_dim, int max_len, float theta,
                    void* stream);

/* The same for a q|k|v projection whose q and k heads come in the row order of the rotary output
 * side of fdk_linear_lut_fused ([0..31, 64..95, 32..63, 96..127] per head; v heads in their own
 * order): for batches that the fused form does not take.  q_out and the caches get the usual order. */
int fdk_rope_append_paired(const void* qkv, const void* pos, void* q_out, void* k_cache, void* v_cache,
                           int rows, int q_heads, int kv_heads, int head_dim, int max_len, float theta,
                           void* stream);

/* out[r] (device int64) = index of the largest of x[r][0 .. n), the lowest index among equals,
 * a NaN counting as the largest: the token choice of the reference's greedy Generator.step
 * (`logits.argmax(dim=-1)`, src/fdk/models.py:252).  x bf16 or fp16, rows of n contiguous. */
int fdk_argmax(const void* x, void* out, int rows, int n, int dtype, void* stream);

/* out[rows, width] = silu(gate) * up, gate_up [rows, 2 width] being the output of the fused
 * gate|up projection, whose columns alternate `group` gate values and the `group` matching up
 * values (group = width: all gates, then all ups; group = 32: the row order that
 * FDK_FLAG_SILU_PAIRS expects).  width must be a multiple of group, group of 8. */
int fdk_silu_mul(const void* gate_up, void* out, int rows, int width, int group, void* stream);

/* Decode attention: one query token per batch row against the static KV cache
 * [batch, kv_heads, max_len, 128] (bf16), keys 0 .. *pos (device int64; the current token's
 * key and value must already be appended), grouped-query (q_heads / kv_heads in 1..8).
 * q, out: [batch, q_heads * 128]; q, the caches and out 16-byte aligned (FDK_ERR_ALIGN).
 * The context is cut into `splits` slices handled by
 * different CTAs; with splits > 1, `scratch` and `counters` of the sizes given by
 * fdk_decode_attention_scratch are needed, BOTH zero-filled once before their first use and
 * then left to the library: the slices hand their sums over as {value, tag} words whose tag
 * is the use count kept in `counters`, so nothing is cleared between calls, and calls that
 * share a scratch must be ordered on one stream.  The last word of `counters` is a status
 * word (fdk_decode_attention_status: 0, or 1 after a bounded wait for a slice ran out; the
 * output of that call is then undefined).  Stands in for the attention of transformers'
 * Llama over its StaticCache (src/fdk/models.py:238-251). */
int fdk_decode_attention_scratch(int batch, int q_heads, int kv_heads, int splits,
                                 size_t* scratch_bytes_host, size_t* counter_bytes_host);
int fdk_decode_attention_status(const void* counters, int batch, int kv_heads, int* status_host);
int fdk_decode_attention(const void* q, const void* k_cache, const void* v_cache, const void* pos,
                         void* out, void* scratch, void* counters, int batch, int q_heads,
                         int kv_heads, int head_dim, int max_len, int splits, void* stream);

/* fdk_linear_lut for a caller whose activations live in HOST memory (the reference's operators
 * take device tensors; a host-side caller would copy around them: x.to(device), the operator,
 * out.cpu()).  One call: x_host [m, k] -> x_dev (asynchronous copy on `stream`), the projection
 * into out_dev, out_dev -> out_host [m, n], and a synchronisation of `stream`: out_host is valid
 * on return (FDK_FLAG_NO_SYNC leaves the synchronisation to the caller).  x_host and out_host should be page-locked for the copies to be asynchronous;
 * x_dev [m, k] and out_dev [m, n] are device staging buffers of the caller (nothing is allocated
 * here); where out_host is page-locked, mapped and 16-byte aligned the projection stores its
 * result straight into it and out_dev is left untouched.  Other arguments as fdk_linear_lut. */
int fdk_linear_lut_host(const void* x_host, const void* tiled, const void* lut, const void* lut_host,
                        void* out_host, int m, int n, int k, int bits, int dtype, void* x_dev, void* out_dev,
                        void* workspace, size_t workspace_bytes, unsigned flags, void* stream);

/* ---- decode-step fusions of fdk_linear_lut (bf16, m <= 16) -------------------------------
 * Around each quantised projection the reference's model (transformers' Llama, called from
 * Generator.step, src/fdk/models.py:245-255) runs an RMSNorm, a residual add or a rotary
 * embedding as separate framework kernels.  Here the projection kernel does them itself:
 *   input side   x = norm_weight * bf16(h * rsqrt(mean(h^2) + eps)) computed while x is staged
 *                (the `x` argument is ignored); mean(h^2) of batch row b is the sum of
 *                norm_sumsq[b][0 .. norm_tiles) divided by k: what the projection that last
 *                updated h left behind (resid_sumsq), or fdk_sumsq_tiles.  x [m, k] must fit in
 *                shared memory beside the kernel's tables (FDK_ERR_SHAPE otherwise).
 *   output side, at most one of
 *     residual   h[m, n] += bf16(y) in place (bf16 add, as the framework model does) instead of
 *                writing `out`; resid_sumsq[b][t] = sum of squares of the new h over rows
 *                64 t .. 64 t + 63 (fp32, fixed order);
 *     rotary     the rows are the fused q|k|v projection, the rows of every q and k head
 *                ordered [0..31, 64..95, 32..63, 96..127] (a pair of the rotate-half formula sits
 *                in one 64-row tile); q is rotated into q_out [m, q_heads * 128], k rotated and v
 *                copied into the caches [m, kv_heads, max_len, 128] at *rope_pos, with the
 *                roundings of fdk_rope_append; rope_table as fdk_rope_table fills it.
 *   FDK_FLAG_SILU_PAIRS may be combined with the input side.
 *   deferred RMSNorm: instead of normalising x while it is staged (which costs ~0.6 us before the
 *                first weight is used), the norm can be split between the projection that writes
 *                the residual stream and the one that reads it.  Producer (residual output with
 *                resid_norm_weight): besides h it writes resid_x = bf16(norm_weight * h).
 *                Consumer (scale_sumsq != NULL; x = that resid_x): every complete sum of batch
 *                row b is multiplied by rsqrt(sum of scale_sumsq[b][0 .. scale_tiles) / k +
 *                scale_eps) before it is rounded and handed to the output side (plain, SiLU,
 *                rotary or residual).  y = inv * (W . (w * h)) equals the norm followed by the
 *                projection up to one bf16 rounding per element of x (w * bf16(h * inv) in the
 *                framework model, bf16(w * h) here).  fdk_norm_prepare makes resid_x and the sums
 *                of squares for a residual stream that no projection has written yet.
 * Results equal the unfused sequence of calls up to the order of the fp32 sum of squares. */
typedef struct fdk_linear_fusion {
  const void* norm_h;       /* [m, k] or NULL */
  const void* norm_weight;  /* [k] */
  const float* norm_sumsq;  /* [m, norm_tiles] */
  int norm_tiles;
  float norm_eps;
  void* resid_h;            /* [m, n] or NULL */
  float* resid_sumsq;       /* [m, ceil(n / 64)] */
  const void* rope_pos;     /* device int64 or NULL */
  const void* rope_table;   /* [64] {bf16 cos, bf16 sin} */
  void* q_out;
  void* k_cache;
  void* v_cache;
  int q_heads, kv_heads, max_len;
  /* deferred RMSNorm (see above): producer side, with resid_h */
  const void* resid_norm_weight; /* [n] or NULL */
  void* resid_x;                 /* [m, n] = bf16(resid_norm_weight * h) */
  /* consumer side */
  const float* scale_sumsq;      /* [m, scale_tiles] or NULL */
  int scale_tiles;
  float scale_eps;
} fdk_linear_fusion;

int fdk_linear_lut_fused(const void* x, const void* tiled, const void* lut, const void* lut_host,
                         void* out, int m, int n, int k, int bits, int dtype, void* workspace,
                         size_t workspace_bytes, unsigned flags, const fdk_linear_fusion* fusion,
                         void* stream);

/* Whether fdk_linear_lut_fused can apply its RMSNorm (norm_h != NULL) to a batch of m rows of k
 * columns: the normalised x has to fit in a CTA's shared memory beside the lookup table
 * (16 rows of 3072 columns do, 16 of 8192 do not).  *fits_host = 1 or 0; shapes the entry point
 * rejects anyway give 0.  The first call on a device asks the device once for the address of
 * its shared window (as fdk_workspace_init does).  No counterpart in the reference. */
int fdk_linear_norm_fits(int m, int k, int bits, int* fits_host);

/* table[i] = {bf16 cos, bf16 sin} of the angle *pos * theta^(-2 i / 128), i = 0 .. 63: once per
 * decode step, for the rotary output side above. */
int fdk_rope_table(const void* pos, void* table, float theta, void* stream);

/* sumsq[b][t] = sum of squares of h[b][64 t .. 64 t + 63] (fp32): the input-side fusion's
 * sums for a residual stream that no projection has written yet (the embedding). */
int fdk_sumsq_tiles(const void* h, float* sumsq, int rows, int width, void* stream);

/* The same sums, and x[b][j] = bf16(weight[j] * h[b][j]): the producer side of the deferred
 * RMSNorm for the first layer of a decode step. */
int fdk_norm_prepare(const void* h, const void* weight, void* x, float* sumsq, int rows, int width,
                     void* stream);

/* fdk_linear_lut for callers that cannot allocate device memory where they call it -- a
 * plugin inside a host runtime that owns all device allocations, or code running while a
 * stream capture forbids cudaMalloc.  Same arguments as fdk_linear_lut minus the workspace, same
 * results (for 17 rows and more up to the order of the fp32 partial sums, the built-in scratch
 * having no room for the tensor-core kernel's split tiles): the scratch is an array inside the library image (1,327,104 bytes, enough for a
 * GPU of up to 160 multiprocessors; a larger GPU is refused with FDK_ERR_WORKSPACE), held by
 * every GPU that loads the library until the process exits.  The call itself allocates
 * nothing, on the host or the device.
 *   - The first call on a device looks up the array's device address and asks the device
 *     where kernels see their shared memory (one one-thread kernel, synchronous): make that
 *     first call before any stream capture.
 *   - All calls on a device share the one array, so two calls that overlap on the GPU
 *     (different streams, no ordering between them) race; serialise them or give the others
 *     fdk_linear_lut with workspaces of their own.  Nothing needs clearing between calls:
 *     the array starts zero-filled and every use of it is tagged.
 * This entry point has no counterpart in the reference. */
int fdk_linear_lut_static(const void* x, const void* tiled, const void* lut, const void* lut_host,
                          void* out, int m, int n, int k, int bits, int dtype, unsigned flags,
                          void* stream);

/* The device-side status word of the built-in scratch of fdk_linear_lut_static on the current
 * device, as fdk_workspace_status reports it for a caller's workspace (synchronous copy of one
 * word; allocates nothing): 0 when every call so far ran normally.  No counterpart in the
 * reference. */
int fdk_static_status(int* status_host);

/* ---- tensor-parallel exchange: row-parallel projection fused with its all-reduce ----------
 * The reference runs on one GPU (its src/ has no collective).  Here a row-parallel projection
 * (o_proj, down_proj: each rank holds a K-slice of the weight and produces a partial sum of
 * the whole output) can store its result straight into every rank's exchange buffer from the
 * kernel's epilogue, and the RMSNorm that follows adds the ranks' partial sums in rank order
 * while it adds the residual: no separate collective launch, one NVLink crossing.
 *
 * Every rank owns one exchange buffer of fdk_tp_exchange_bytes(tp, slot_elems) bytes, zeroed,
 * and maps the buffers of the others (fdk_tp_buffer_*: CUDA IPC, all ranks on one node with
 * peer access).  It holds two halves used alternately, each with one slot per rank of
 * slot_elems partial sums, stored as 8-byte words {two 16-bit values, 32-bit tag}, and this
 * rank's count of completed reduces.  A word is valid for the reduce once its tag is the
 * number of the push, so a push needs no fence, flag or acknowledgement: one crossing of the
 * link.  Rules:
 *   - all ranks make the same sequence of push / reduce calls, each push followed by its
 *     reduce on the same stream before the next push (the decode loop does);
 *   - m <= 16, n a multiple of 64, m * n <= slot_elems;
 *   - only plain stores to peer memory are used: no multicast of any kind.
 * A reduce waits at most two seconds for a word of another rank, then records status 1 in
 * the buffer (fdk_tp_exchange_status), takes the word as zero and carries on. */
#define FDK_TP_MAX_RANKS 8
typedef struct fdk_tp_exchange {
  int tp;                          /* ranks, 1..FDK_TP_MAX_RANKS */
  int rank;                        /* this rank */
  void* buffers[FDK_TP_MAX_RANKS]; /* every rank's exchange buffer as mapped here; buffers[rank] is this rank's */
  long long slot_elems;            /* 16-bit elements per slot, a multiple of 8 */
} fdk_tp_exchange;

size_t fdk_tp_exchange_bytes(int tp, long long slot_elems);
/* Allocates `bytes` of zeroed device memory on the current device and writes its 64-byte IPC
 * handle; the other ranks pass the handle to fdk_tp_buffer_open (which enables peer access)
 * and later to fdk_tp_buffer_close; the owner frees with fdk_tp_buffer_destroy. */
int fdk_tp_buffer_create(size_t bytes, void** ptr_host, unsigned char* handle_host);
int fdk_tp_buffer_open(const unsigned char* handle_host, void** ptr_host);
int fdk_tp_buffer_close(void* ptr);
int fdk_tp_buffer_destroy(void* ptr);
int fdk_tp_exchange_status(const fdk_tp_exchange* ex, int* status_host);

/* fdk_linear_lut whose output [m, n] goes to slot `rank` of the current half of every rank's
 * exchange buffer instead of `out`, each CTA storing the rows it finishes. */
int fdk_linear_lut_push(const void* x, const void* tiled, const void* lut, const void* lut_host,
                        int m, int n, int k, int bits, int dtype, void* workspace,
                        size_t workspace_bytes, unsigned flags, const fdk_tp_exchange* ex,
                        void* stream);

/* fdk_rmsnorm whose `delta` is the sum over ranks (fp32, in rank order, rounded to bf16) of the
 * partial sums of the latest push, each word waited for as it is needed.  rows, width must be
 * the m, n of that push. */
int fdk_rmsnorm_reduce(void* h, const fdk_tp_exchange* ex, const void* weight, void* out, int rows,
                       int width, float eps, void* stream);

#ifdef __cplusplus
}
#endif
#endif /* FDK_B200_H_ */

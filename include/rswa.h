/* rswa.h -- C ABI of the B200 (sm_100a) ring sliding-window attention kernels.
 *
 * Plain pointers and sizes only.  Every buffer, workspace included, is owned by the caller;
 * all work is enqueued on the stream passed in; nothing here allocates device memory (except
 * where an entry point says otherwise) and nothing synchronises the device.  Entry points
 * return 0 on success and a negative RSWA_E_* code on a rejected argument; rswa_last_error()
 * gives the message for the calling thread.
 *
 * What each entry point replaces in the reference (paths are inside the reference project):
 * the reference reaches its arithmetic through four Python wrappers around the flash-attn
 * custom ops and one Triton merge kernel; the entry points below are what a maintainer binds
 * instead (from Python with ctypes, as ring_swa/_C.py does).
 */
#ifndef RSWA_H_
#define RSWA_H_

#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

#define RSWA_ABI_VERSION 1
#define RSWA_MAX_SPANS 10
#define RSWA_TILE 128 /* query rows and key rows per tile */

#define RSWA_DTYPE_BF16 0
#define RSWA_DTYPE_FP16 1
#define RSWA_DTYPE_F32 2 /* only where an entry point says float is accepted */

#define RSWA_OK 0
#define RSWA_E_ARG (-1)      /* bad shape / stride / alignment / null pointer */
#define RSWA_E_UNSUPPORTED (-2)
#define RSWA_E_CUDA (-3)     /* a CUDA runtime/driver call failed at launch time */
#define RSWA_E_NOALLOC_SIZE (-4) /* rswa_bwd_noalloc: the problem does not fit the built-in scratch */

/* size of the scratch array inside the library that rswa_bwd_noalloc works in: 64 MiB for the two
 * float rows per (batch row, head, token) plus the 256 bytes of work counters every backward
 * workspace ends with */
#define RSWA_NOALLOC_SCRATCH_BYTES ((64ll << 20) + 256)

/* bits of rswa_bwd_params_t.flags */
#define RSWA_BWD_INIT 1   /* fill the workspace rows: delta = rowsum(dO*O) and lse*log2(e) */
#define RSWA_BWD_FINISH 2 /* also compute dq, summed over ALL spans of this call */

/* A span is a run of consecutive tokens' K and V (and, in backward, their gradients) that sits
 * in one buffer: the rank's own tokens, a halo received from an earlier rank, or the sink
 * tokens received from the owner of the sequence start.  Spans of one call must not overlap in
 * position.  Layout [batch, len, n_kv_heads, head_dim], strides in elements, head_dim
 * contiguous. */
typedef struct rswa_span {
  const void* k;
  const void* v;
  void* dk; /* backward only; bf16/fp16 like k, or float when grad_fp32 != 0 */
  void* dv;
  int64_t kv_stride_b, kv_stride_t, kv_stride_h;     /* k and v share strides */
  int64_t dkv_stride_b, dkv_stride_t, dkv_stride_h;  /* dk and dv share strides */
  int32_t pos_start; /* global position of the span's first token */
  int32_t len;       /* tokens */
  int32_t grad_fp32;
  int32_t reserved;
} rswa_span_t;

/* Shared geometry.  A query at global position p sees key t iff both lie in the same sequence,
 * t <= p, and (p - t <= window  or  t < seq_start(p) + n_sink).  Sequences are the batch rows
 * when cu_seqlens is NULL, else the segments of the packed token axis given by the GLOBAL
 * cumulative lengths (int32, device memory, n_seqs + 1 entries) and batch must be 1. */
typedef struct rswa_geom {
  int32_t dtype;
  int32_t batch, q_len, n_q_heads, n_kv_heads, head_dim; /* head_dim must be 128 */
  int32_t q_pos_start; /* global position of local query 0 */
  int32_t window, n_sink;
  float softmax_scale;
  const int32_t* cu_seqlens;
  int32_t n_seqs;
  int32_t n_spans;
  rswa_span_t spans[RSWA_MAX_SPANS];
} rswa_geom_t;

/* Forward: out [batch,q_len,Hq,D] and lse [batch,Hq,q_len] (natural log, fp32; -inf and a zero
 * output row where no key of the given spans is visible).  Only query tiles
 * [q_tile_begin, q_tile_end) are computed (q_tile_end <= 0: all).
 * With `carry` the call continues a partial result instead of starting a new one.
 * Replaces wrapped_flash_attn_fwd / wrapped_flash_attn_fwd_varlen
 * (ring_swa/ops/wrap_flash.py:168-200, 203-273) and the per-hop mask-case selection around them
 * (ring_swa/sliding_window/nonvarlen.py:95-150, ring_swa/ops/attn.py:12-60). */
typedef struct rswa_fwd_params {
  rswa_geom_t g;
  const void* q;
  int64_t q_stride_b, q_stride_t, q_stride_h;
  void* out;
  int64_t o_stride_b, o_stride_t, o_stride_h;
  float* lse;
  int64_t lse_stride_b, lse_stride_h;
  int32_t q_tile_begin, q_tile_end;
  int32_t* status; /* device word; set non-zero if a device-side wait ran out */
  /* non-zero: out / lse already hold a partial result over OTHER keys (an earlier call with other
   * spans); this call continues it -- running maximum and weight start from lse, the accumulator from
   * out -- and overwrites both with the combined result, as merge_attn_out would have combined two
   * partial results (ring_swa/ops/attn.py:31-36, ring_swa/ops/merge.py:68-147).  Rows that see no key of
   * this call's spans keep what they hold. */
  int32_t carry;
  int32_t reserved;
} rswa_fwd_params_t;

int rswa_fwd(const rswa_fwd_params_t* p, void* stream);

/* Backward: dq [batch,q_len,Hq,D] and per-span dk/dv from (dO, q, spans, out, lse), using the
 * final (merged) out and lse.  Two kernels: a key-stationary one writes dk/dv of every span that
 * carries dk/dv pointers (spans with both NULL take part in dq only), a query-stationary one
 * writes dq summed over all spans of the call when FINISH is set.  Nothing is reduced through
 * global memory, so the result is deterministic.  `workspace` is rswa_bwd_workspace_bytes() of
 * device memory (two fp32 rows per batch row and head: delta and the scaled lse, filled by INIT; plus
 * 256 bytes for the work counter of the dQ kernel, which the call itself resets on the stream).
 * One call with flags INIT|FINISH does a whole backward.  A ring rank calls it twice with the same
 * workspace: INIT with the received spans only (their gradients can leave early), then FINISH with
 * every span, gradient pointers on the local one only.
 * Replaces wrapped_flash_attn_bwd / wrapped_flash_attn_bwd_varlen
 * (ring_swa/ops/wrap_flash.py:276-327, 330-429) and ring_swa/ops/attn.py:63-126. */
typedef struct rswa_bwd_params {
  rswa_geom_t g;
  const void* q;
  int64_t q_stride_b, q_stride_t, q_stride_h;
  const void* out;
  int64_t o_stride_b, o_stride_t, o_stride_h;
  const void* dout;
  int64_t do_stride_b, do_stride_t, do_stride_h;
  const float* lse;
  int64_t lse_stride_b, lse_stride_h;
  void* dq;
  int64_t dq_stride_b, dq_stride_t, dq_stride_h;
  void* workspace;
  int64_t workspace_bytes;
  int32_t flags;
  int32_t* status;
  /* Optional hooks: events from rswa_event_create(), recorded on the stream right before and
   * right after the two tensor-core kernels (the delta kernel excluded).  NULL to skip.
   * ev_main_mid is recorded between the dK/dV kernel and the dQ kernel: besides timing, another
   * stream may wait for it (rswa_event_wait) and pick the K/V gradients up while dQ is computed;
   * a ring rank sends the received spans' gradients back that way. */
  void* ev_main_start;
  void* ev_main_stop;
  void* ev_main_mid;
} rswa_bwd_params_t;

int64_t rswa_bwd_workspace_bytes(int32_t batch, int32_t q_len, int32_t n_q_heads, int32_t head_dim);
int rswa_bwd(const rswa_bwd_params_t* p, void* stream);

/* The whole backward for callers that cannot allocate device memory: same inputs, outputs and
 * result as rswa_bwd with flags INIT|FINISH, but `workspace`, `workspace_bytes` and `flags` are
 * ignored.  The scratch (the delta and scaled-lse rows the kernels read) is a fixed array of
 * RSWA_NOALLOC_SCRATCH_BYTES that is part of the library's device image, so every GPU that loads
 * the library carries it until the process exits, and the call itself never allocates or frees.
 * Meant for hosts that are handed only the operator's tensors (a plugin inside another runtime),
 * that gave away all device memory at start-up, or that must not stall their other streams with
 * the device-wide synchronisation an allocation implies.
 *  - rswa_bwd_workspace_bytes(batch, q_len, n_q_heads, 128) must not exceed
 *    RSWA_NOALLOC_SCRATCH_BYTES (batch * n_q_heads * q_len padded to whole tiles <= 8388608 rows:
 *    262144 tokens of 32 heads just fit); larger problems return RSWA_E_NOALLOC_SIZE and launch nothing.
 *  - The first call on each device looks the array's device address up (with that device
 *    current).  Make that first call outside any stream capture.
 *  - All calls on a device share the array: it is rewritten at the start of each call, and
 *    two calls that can overlap on the GPU (different streams, no dependency) corrupt each other.
 * Has no counterpart in the reference, whose backward allocates its accumulators with torch on
 * every call (ring_swa/sliding_window/nonvarlen.py:192-195). */
int rswa_bwd_noalloc(const rswa_bwd_params_t* p, void* stream);
int64_t rswa_noalloc_scratch_bytes(void);

/* Log-sum-exp merge of two partial results over the same queries:
 *   lse = log(exp(lse_a) + exp(lse_b)),  o = o_a*exp(lse_a-lse) + o_b*exp(lse_b-lse)
 * o_* are [rows, D] 16-bit with a row stride (rows = batch*q_len*Hq flattened by the caller's
 * strides below), lse_* fp32.  In place (o == o_a, lse == lse_a) is allowed.  (-inf,-inf) gives
 * (0,-inf).  Replaces merge_attn_out (ring_swa/ops/merge.py:150-193, kernel :68-147). */
typedef struct rswa_merge_params {
  int32_t dtype;
  int32_t batch, q_len, n_heads, head_dim;
  const void* o_a;
  const void* o_b;
  void* o;
  int64_t oa_stride_b, oa_stride_t, oa_stride_h;
  int64_t ob_stride_b, ob_stride_t, ob_stride_h;
  int64_t o_stride_b, o_stride_t, o_stride_h;
  const float* lse_a;
  const float* lse_b;
  float* lse; /* all three [batch, n_heads, q_len] with the strides below */
  int64_t lse_stride_b, lse_stride_h;
} rswa_merge_params_t;

int rswa_merge(const rswa_merge_params_t* p, void* stream);

/* The same merge, in place into the higher-precision accumulators the reference carries between
 * ring hops: acc_o float [batch,q_len,n_heads,head_dim] (strided views allowed), acc_lse float or
 * double [batch,n_heads,q_len]; the incoming partial result is bf16, fp16 or float with a float
 * lse.  The lse is combined in float whatever the accumulator holds, as the reference's kernel does
 * (ring_swa/ops/merge.py:134-135).  An accumulator lse of -inf gives the incoming result exactly.
 * head_dim: any multiple of 4.  Replaces merge_attn_out as called from flash_attn_fwd_func
 * (ring_swa/ops/attn.py:31-36) and from the ring loops (ring_swa/sliding_window/nonvarlen.py:95-150). */
typedef struct rswa_merge_acc_params {
  int32_t new_dtype; /* RSWA_DTYPE_BF16, RSWA_DTYPE_FP16 or RSWA_DTYPE_F32 */
  int32_t lse_f64;   /* accumulator lse: 0 = float, 1 = double */
  int32_t batch, q_len, n_heads, head_dim;
  float* acc_o;
  int64_t acc_stride_b, acc_stride_t, acc_stride_h;
  const void* new_o;
  int64_t new_stride_b, new_stride_t, new_stride_h;
  void* acc_lse;
  int64_t acc_lse_stride_b, acc_lse_stride_h; /* tokens contiguous */
  const float* new_lse;
  int64_t new_lse_stride_b, new_lse_stride_h;
} rswa_merge_acc_params_t;

int rswa_merge_acc(const rswa_merge_acc_params_t* p, void* stream);

/* acc[b, t, :] += recv[b, t, :] for a [batch, len, row] block: adds the K/V gradients a later
 * rank computed for this rank's trailing tokens (the halo) into the fp32 accumulator.
 * recv_dtype: RSWA_DTYPE_* or 2 for float.  Replaces the dkv.add_ of the reverse ring
 * (ring_swa/sliding_window/nonvarlen.py:313-322). */
int rswa_halo_accumulate(float* acc, int64_t acc_stride_b, const void* recv, int64_t recv_stride_b,
                         int32_t recv_dtype, int32_t batch, int64_t elems_per_batch, void* stream);

/* dst (16-bit) = round(acc + recv), acc itself left untouched: the last of the additions above and the
 * final cast (ring_swa/sliding_window/nonvarlen.py:320-322, 335-337) in one pass over the data.
 * dst_dtype: RSWA_DTYPE_BF16 or RSWA_DTYPE_FP16; recv_dtype as for rswa_halo_accumulate. */
int rswa_halo_accumulate_cast(void* dst, int64_t dst_stride_b, int32_t dst_dtype, const float* acc,
                              int64_t acc_stride_b, const void* recv, int64_t recv_stride_b, int32_t recv_dtype,
                              int32_t batch, int64_t elems_per_batch, void* stream);

/* dst (16-bit) = src (float), [batch, elems_per_batch] with batch strides: the final cast of
 * ring_swa/sliding_window/nonvarlen.py:335-337. */
int rswa_cast_from_f32(void* dst, int64_t dst_stride_b, const float* src, int64_t src_stride_b,
                       int32_t dtype, int32_t batch, int64_t elems_per_batch, void* stream);

/* Peer-store halo exchange between the GPUs of one node (buffers in memory the receiver owns and the
 * sender has mapped, e.g. torch symmetric memory; this library maps nothing itself).
 * rswa_peer_put: copy `rows` rows of `row_bytes` bytes from src (local) to dst (local or a peer's), with
 * the given pitches, on the copy engines (no kernel, no SM), then, if flag is non-NULL, release `value`
 * into *flag (local or a peer's) from a one-thread kernel behind the copy on the same stream.
 * rswa_flag_set: that release alone (an acknowledgement).
 * rswa_flag_wait: a one-thread kernel that returns once *flag (local memory) has reached `value`
 * (numbers only grow; wrap-safe) -- what is launched behind it on the stream then finds the data the
 * number announces -- or, after timeout_ns, sets *status to a non-zero code and returns.
 * Replaces ring_attn_p2p_communicate (ring_swa/ops/comm.py:8-40: NCCL isend / irecv per hop). */
int rswa_peer_put(void* dst, int64_t dst_pitch, const void* src, int64_t src_pitch, int64_t row_bytes,
                  int64_t rows, int32_t* flag, int32_t value, void* stream);
int rswa_flag_set(int32_t* flag, int32_t value, void* stream);
int rswa_flag_wait(const int32_t* flag, int32_t value, int32_t* status, int64_t timeout_ns, void* stream);

/* One 128x128x128 tensor-core product through each operand path the attention kernels use
 * (shared-memory K-major / MN-major operands, tensor-memory A operand); for the unit tests.
 * a, b: bf16 [128,128] row-major device buffers; d: float [128,128].
 *   mode 0: d = a * b^T      (both K-major)
 *   mode 1: d = a * b        (B MN-major)
 *   mode 2: d = a * b        (A through tensor memory, B MN-major)
 *   mode 3: d = a^T * b      (A and B MN-major)
 * No counterpart in the reference. */
int rswa_selftest_mma(int32_t mode, const void* a, const void* b, float* d, int32_t* status,
                      void* stream);

/* Events (thin wrappers of cudaEvent_t so that callers need no CUDA headers): timing for benchmarks,
 * and ordering between streams.  No counterpart in the reference, which times with torch.cuda.Event
 * (test/test_ring_swa_nonvarlen.py:295-320). */
void* rswa_event_create(void);
void rswa_event_destroy(void* ev);
int rswa_event_record(void* ev, void* stream);
/* work queued on `stream` after this call starts once the event's latest record has completed */
int rswa_event_wait(void* ev, void* stream);
/* milliseconds between two recorded events, after synchronising on `stop`; negative on error */
float rswa_event_elapsed_ms(void* start, void* stop);

int rswa_abi_version(void);
const char* rswa_last_error(void);

#ifdef __cplusplus
}
#endif
#endif /* RSWA_H_ */

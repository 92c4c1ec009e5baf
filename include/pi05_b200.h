/* C ABI of the B200 pi0.5 action-chunk engine.
 *
 * One handle = one engine on one GPU.  Every pointer is a plain device (or, where stated, host)
 * pointer; no framework types cross this boundary.  Every function returns a PI05_* status code;
 * argument errors are detected on the host and never touch the GPU.  Handles hold all state, so
 * several handles (one per GPU) can live in one process.
 *
 * The entry points replace, one for one, the native interface of the reference's megakernel arm
 * (mk/pi05_mk.cu:3658-3670: setup / workspace_bytes / launch / layout_offsets / build_config /
 * fg_timeouts / att_timeouts) as it is driven by megakernel.py:117-186.
 */
#ifndef PI05_B200_H_
#define PI05_B200_H_

#include <stddef.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

typedef struct pi05_engine* pi05_handle_t;

enum {
  PI05_OK = 0,
  PI05_ERR_ARGUMENT = 1,      /* null pointer, bad size, misaligned buffer, bad handle */
  PI05_ERR_UNSUPPORTED = 2,   /* geometry / batch / tensor-parallel setting not built */
  PI05_ERR_CUDA = 3,          /* a CUDA runtime or driver call failed (see pi05_last_error) */
  PI05_ERR_NOT_BOUND = 4,     /* launch before bind */
  PI05_ERR_DEVICE_TIMEOUT = 5,/* a bounded device-side wait gave up; see pi05_status */
  PI05_ERR_NO_DEVICE = 6      /* no usable sm_100 GPU */
};

/* Number of input tensors and their fixed order (reference megakernel.py:21-25):
 *  0 action_in_weight [1024,32] f32     1 action_in_bias [1024] f32
 *  2 time_in_weight [1024,1024] f32     3 time_in_bias [1024] f32
 *  4 time_out_weight [1024,1024] f32    5 time_out_bias [1024] f32
 *  6 action_out_weight [32,1024] f32    7 action_out_bias [32] f32
 *  8 wq [18,2048,1024] bf16   9 wk [18,256,1024] bf16  10 wv [18,256,1024] bf16
 * 11 wo [18,1024,2048] bf16  12 wg [18,4096,1024] bf16 13 wu [18,4096,1024] bf16
 * 14 wd [18,1024,4096] bf16
 * 15 attn_norm_weight [18,3072,1024] f32  16 attn_norm_bias [18,3072] f32
 * 17 ffn_norm_weight  [18,3072,1024] f32  18 ffn_norm_bias  [18,3072] f32
 * 19 final_norm_weight [3072,1024] f32    20 final_norm_bias [3072] f32
 * 21 noise [50,32] f32   22 prefix_k [18,P,1,256] bf16   23 prefix_v [18,P,1,256] bf16
 * 24 prefix_mask [P] bool (one byte per token, non-zero = valid)
 * With a batch of B > 1 observations, tensors 21-24 (and the actions output) carry a leading index [B, ...]:
 * every observation has its own noise, prefix cache and mask; tensors 0-20 (the weights) are shared.          */
#define PI05_NUM_INPUTS 25

/* Replaces setup(device) (mk/pi05_mk.cu:3363-3380).  max_prefix bounds the prefix length accepted by
 * pi05_bind; max_batch (1..16) is the largest number of independent observations one launch may serve (the
 * workspace grows with it; the weights are streamed from HBM once per launch for all of them); tp_rank and
 * tp_size (1, 2, 4 or 8; more than 1 only with max_batch = 1) make this engine one of tp_size ranks, one per GPU,
 * that share a single observation: see "tensor parallel" below. */
int pi05_create(int device, int max_prefix, int max_batch, int tp_rank, int tp_size, pi05_handle_t* out);

/* Tuning settings of a handle: the counterpart of the reference's build variants and -D macros (megakernel.py:29-78,
 * mk/pi05_mk.cu:34-320), as run-time values.  The library reads no environment variable; a host program that wants
 * settings from its environment fills this struct itself.  pi05_tuning_defaults writes the values a fresh handle
 * uses; pi05_tune replaces a handle's settings (values out of range are clamped) and un-binds it: the schedule and
 * the launch shape are chosen by the next pi05_bind. */
typedef struct pi05_tuning {
  int poll_ns;            /* pause between two samples of a stage counter (default 20) */
  int obs_per_mma;        /* observations side by side in one MMA of a batch: 0 = engine's choice, 1, 2 */
  int two_streams;        /* batches: the throughput schedule as two streams of groups half a layer pass apart (default 1) */
  int entries_per_phase;  /* batches: schedule entries per CTA and phase the K splits aim at; 0 = by batch size */
  int grouped_from;       /* smallest batch that gets the throughput schedule (default 3) */
  int streams_from;       /* smallest batch that gets its two streams (default 5) */
  int latency_schedule;   /* 1: the one-observation schedule for every batch size (default 0) */
  int key_groups;         /* one observation: groups of row CTAs that share the keys of an attention; 0 = by prefix length */
  int row_groups;         /* batches: groups of row CTAs; 0 = by batch size */
  int clusters;           /* launch the grid as clusters of two CTAs when the device takes it that way (default 1) */
  int cta_perm;           /* 1: the two blocks of a cluster play CTA i and CTA grid / 2 + i (default 0) */
} pi05_tuning;
int pi05_tuning_defaults(pi05_tuning* t);
int pi05_tune(pi05_handle_t h, const pi05_tuning* t);

/* Replaces workspace_bytes() (mk/pi05_mk.cu:3659-3660): size of the scratch buffer the caller allocates
 * on the engine's GPU (256-byte aligned) and passes to pi05_bind. */
int pi05_workspace_bytes(pi05_handle_t h, size_t* bytes);

/* Replaces the tensor-list half of launch() (mk/pi05_mk.cu:3523-3557) and MegakernelArm.bind
 * (megakernel.py:167-176): records the 25 device pointers (caller-owned, read-only, kept across launches and
 * across in-place refills), the output buffer actions [50,32] f32 and the workspace, clears the workspace and
 * encodes the TMA descriptors.  prefix_len is P (1..max_prefix), batch the number of observations (1..max_batch).
 * Waits for the handle's last launch (a re-bind must not pull the workspace from under a running chunk) and
 * synchronises the device. */
int pi05_bind(pi05_handle_t h, const void* const inputs[PI05_NUM_INPUTS], int prefix_len, int batch,
              void* actions, void* workspace, size_t workspace_bytes);

/* The prefix cache where its producer left it (the hand-off after `prefill`, reference/pi05.py:167-195, whose keys
 * and values the reference passes on as dense [18,P,1,256] tensors): a pool of pages with arbitrary strides, and per
 * observation a list of the pages that hold its tokens in order.  Nothing is copied or repacked; the attention's
 * tiled copies read the pool through these strides.
 *   token t of observation b, layer l, lives at
 *     k + (page_table[b * pages_per_obs + t / page_tokens] * page_stride + l * layer_stride
 *          + (t % page_tokens) * token_stride) elements, 256 contiguous BF16 from there (v likewise).
 * Requirements: k and v 16-byte aligned; the three strides multiples of 8 elements; page_tokens a multiple of 64
 * unless pages_per_obs is 1 (one page per observation: any length >= prefix_len, e.g. a cache allocated for the
 * longest prompt and filled up to prefix_len); prefix_len <= pages_per_obs * page_tokens; every page_table entry in
 * [0, num_pages).  page_table is a host array and is copied at bind time.  Tokens at and beyond prefix_len are never
 * read as values: whatever the cache holds there cannot reach the result. */
typedef struct pi05_kv_view {
  const void* k;
  const void* v;
  long long token_stride, layer_stride, page_stride;   /* in BF16 elements */
  int page_tokens;
  int num_pages;
  int pages_per_obs;
  const int* page_table;
} pi05_kv_view;

/* pi05_bind with the prefix cache given as a view: inputs[22] and inputs[23] are ignored (may be NULL), everything
 * else is as in pi05_bind (inputs[24], the validity mask, stays [batch][prefix_len]).  pi05_bind itself is this call
 * with the dense view (one page per observation, token stride 256, layer stride prefix_len * 256). */
int pi05_bind_view(pi05_handle_t h, const void* const inputs[PI05_NUM_INPUTS], const pi05_kv_view* kv, int prefix_len,
                   int batch, void* actions, void* workspace, size_t workspace_bytes);

/* Counterpart of the harness's optional refresh_weights() (bench.py:209-216).  The engine reads the caller's
 * tensors in place and keeps no repacked copies, so this only re-validates the binding. */
int pi05_refresh(pi05_handle_t h);

/* Replaces launch() (mk/pi05_mk.cu:3523-3620): one whole action chunk, asynchronous on `stream` (a cudaStream_t;
 * NULL = default stream).  n_steps <= 10 Euler steps and n_layers <= 18 expert layers are run (dt stays -0.1);
 * the graded chunk is (10, 18).  stamps, if non-NULL, is a device buffer of PI05_NUM_STAMPS uint64 that
 * receives globaltimer values at stage boundaries of the first layer passes and, from three GEMM CTAs, at the
 * points of their pipeline in the second pass (the reference's tstamp tensor, mk/pi05_mk.cu:351).  The caller
 * zeroes it. */
int pi05_launch(pi05_handle_t h, int n_steps, int n_layers, void* stream, unsigned long long* stamps);
#define PI05_NUM_STAMPS 256

/* Replaces fg_timeouts()/att_timeouts() (mk/pi05_mk.cu:3505-3520): waits for this handle's last launch (not for the
 * whole device: other handles and streams keep running) and reads the status word the kernel writes when a bounded
 * wait gives up.  code = 0 when the last launches completed; otherwise code is a PI05_WAIT_* value and where =
 * (cta << 16) | stage, PI05_ERR_DEVICE_TIMEOUT is returned, and the word is cleared.  A chunk whose wait gave up has
 * filled its actions with NaN, so a caller that skips this call cannot take an earlier chunk's result for this one's.
 * pi05_launch itself does not look at the word. */
int pi05_status(pi05_handle_t h, int* code, int* where);

/* Replaces layout_offsets() (mk/pi05_mk.cu:3622-3627): byte offset and size of a named workspace buffer
 * ("mod", "cond", "h", "an_attn", "an_ffn", "qkv_acc", "k", "v", "attn", "o_acc", "act", "d_acc", "x", "rope", ...)
 * for stage-by-stage checks. */
int pi05_workspace_region(pi05_handle_t h, const char* name, size_t* offset, size_t* bytes);

/* Debug control: run only the first max_stage stages after the prologue (a stage is one of the seven
 * per-layer steps QKV, attention, O, residual+norm, gate/up, down, residual+norm); negative = run everything.
 * wait_limit_cycles > 0 overrides the bound (in SM clock cycles) of every device-side wait.  drop_event >= 0
 * makes the row CTAs skip that stage-completion signal (PI05_EVENT_*), so that the waits on it run out: the
 * way to exercise the time-out path without stalling a GPU; negative = signal everything. */
int pi05_debug(pi05_handle_t h, int max_stage, long long wait_limit_cycles, int drop_event);
#define PI05_EVENT_ATTENTION_DONE 7
#define PI05_EVENT_FFN_NORM_READY 9
/* pi05_status codes: which kind of wait gave up */
#define PI05_WAIT_WEIGHT_SLOT 1
#define PI05_WAIT_WEIGHT_DATA 2
#define PI05_WAIT_ACT_SLOT 3
#define PI05_WAIT_ACT_DATA 4
#define PI05_WAIT_TMEM_SLOT 5
#define PI05_WAIT_TMEM_DATA 6
#define PI05_WAIT_EVENT 7
#define PI05_WAIT_DRAIN 8

/* Replaces build_config() (mk/pi05_mk.cu:3632-3656): a JSON object describing the build and the schedule. */
const char* pi05_config_json(pi05_handle_t h);

/* The work schedule the engine would bind for `batch` observations of `prefix_len` prefix tokens on a GPU of `sms`
 * SMs, computed on the host without touching a device (the reference derives each block's K chunk and
 * tiles from blockIdx inside its GEMM phases, mk/pi05_mk.cu:736-743, and has no such query; this one exists so that the schedule's invariants can be tested
 * without a GPU).  Writes up to `capacity` entries of PI05_PLAN_ENTRY ints, in the order the CTAs execute them:
 * {cta, gemm (0 QKV, 1 O, 2 gate/up, 3 down), lag (1: the entry belongs to the layer pass before the cycle's),
 * group of observations (-1: every group in turn), tile, first 128-k stage, number of stages}; and info =
 * {GEMM CTAs, row-CTA groups, key groups, observations per MMA, groups of observations, groups in the first of two
 * streams (0: one stream), units per observation of QKV, O, gate/up, down}.  *count receives the number of entries
 * there are, which may exceed capacity.  tuning = NULL: the defaults of a fresh handle. */
#define PI05_PLAN_ENTRY 7
#define PI05_PLAN_INFO 10
int pi05_schedule_plan(int sms, int batch, int prefix_len, const pi05_tuning* tuning, int* entries, int capacity,
                       int* count, int info[PI05_PLAN_INFO]);

/* Tensor parallel (no counterpart in the reference, which runs on one GPU only): tp_size engines, one per GPU, each
 * bound to the SAME 25 inputs in its own GPU's memory, compute one chunk together.  Rank r streams only its share of
 * the weights - query heads 8 r / tp_size .. of wq (and the matching columns of wo), MLP columns 4096 r / tp_size ..
 * of wg / wu (and the matching columns of wd), as reference/pi05.py:254-265 and 268-279 would be cut; wk / wv and the
 * single KV head, the norms and the small FP32 layers run on every rank - and after the O and the down projection
 * every rank stores its [50, 1024] FP32 partial sums into a receive buffer in every PEER's workspace with plain
 * stores over NVLink, bumps a counter there (release at system scope), waits (bounded) for its own counters and adds
 * the partial sums in rank order, so that all ranks keep the same residual stream and every rank's actions buffer
 * receives the result.  Set-up, after every rank has bound its inputs: exchange the pi05_tp_export blobs between the
 * ranks (any host transport), pi05_tp_attach each peer's blob, make sure every rank has attached (a host barrier),
 * then launch the same (n_steps, n_layers) on every rank.  A rank whose peer never arrives reports
 * PI05_ERR_DEVICE_TIMEOUT through pi05_status like any other bounded wait; all ranks then have to bind again.
 * pi05_tp_attach_pointer takes the peer's workspace address directly (one process that drives several GPUs with
 * peer access enabled). */
#define PI05_TP_HANDLE_BYTES 96
int pi05_tp_export(pi05_handle_t h, void* out, size_t out_bytes);
int pi05_tp_attach(pi05_handle_t h, int peer_rank, const void* exported);
int pi05_tp_attach_pointer(pi05_handle_t h, int peer_rank, void* peer_workspace);
/* pi05_schedule_plan for rank tp_rank of tp_size. */
int pi05_schedule_plan_tp(int sms, int batch, int prefix_len, int tp_rank, int tp_size, const pi05_tuning* tuning,
                          int* entries, int capacity, int* count, int info[PI05_PLAN_INFO]);

/* Number of kernel launches issued by this handle since creation (one per pi05_launch). */
int pi05_launch_count(pi05_handle_t h, unsigned long long* count);

const char* pi05_error_string(int code);
const char* pi05_last_error(pi05_handle_t h);

int pi05_destroy(pi05_handle_t h);

/* One whole chunk without any device allocation by anybody.  (No counterpart in the reference: its arm always
 * receives a torch-allocated workspace.)
 *
 * For callers that cannot obtain device memory at the point where they need the engine: code running under an
 * allocator that is frozen or owned by someone else (a memory pool sized up front, a plugin called from inside
 * another framework's execution step, a process that has handed all remaining memory to a cache), where a
 * cudaMalloc would fail, deadlock with the owner's bookkeeping, or is simply forbidden.  The caller passes only
 * the 25 inputs (same order, shapes and alignment as pi05_bind) and the output buffer actions [50,32] f32; the
 * engine's workspace is a fixed array of PI05_STATIC_SCRATCH_BYTES inside the library's device image.  That
 * array exists once per GPU, is held from library load to process exit, and is shared by every call on that
 * GPU: it keeps the previous call's contents (the entry point re-zeroes the control words it needs on the
 * stream before launching), and two calls that overlap on the same GPU - different streams, different host
 * threads - race on it and give wrong results; issue them on one stream or order them yourself.
 *
 * The first call on a device does the set-up (host-side state with one event and one small stream, address of the
 * array, shared-memory opt-in), and the first call with a given set of pointers / prefix length encodes the TMA
 * descriptors and clears the array after waiting for the previous call out of the array, on whatever stream that
 * was; both synchronise the device, so make that call once before any stream capture or latency-critical region.
 * A device-side wait that gave up cannot be reported by the asynchronous call that hit it: the kernel then fills
 * actions with NaN, and the NEXT call on that GPU that finds the earlier kernel finished returns
 * PI05_ERR_DEVICE_TIMEOUT instead of launching (call again to go on).
 * Later calls with the same pointers only enqueue a memset of the control block (about 30 KB) and the kernel on `stream`.  No cudaMalloc,
 * cudaFree or allocating library routine is called on any of these paths.
 *
 * Limits: prefix_len <= PI05_STATIC_MAX_PREFIX and a GPU whose schedule fits the array (any B200), otherwise
 * PI05_ERR_UNSUPPORTED; batch 1 only.  Returns a PI05_* code; the call is asynchronous like pi05_launch. */
#define PI05_STATIC_SCRATCH_BYTES (12u << 20)
#define PI05_STATIC_MAX_PREFIX 1024
int pi05_chunk_static(int device, const void* const inputs[PI05_NUM_INPUTS], int prefix_len, void* actions,
                      int n_steps, int n_layers, void* stream);

/* ---- Gemma-2B prefix prefill: the step before the action chunk.
 * Replaces the reference's eager `prefill(case, values, embeddings, valid)` (reference/pi05.py:167-195), which its
 * fixture runs to obtain the per-layer key / value cache (fixture.py:66-81): RMSNorm, q / k / v projections with RoPE at
 * the positions of the valid tokens, bidirectional attention among valid tokens, O projection, GeGLU MLP, 18 layers
 * (the last layer's MLP is skipped: it affects no cached key or value).  Outputs are the post-RoPE keys and the values,
 * [18, tokens, 1, 256] BF16 - exactly inputs 22 and 23 of pi05_bind, so the chunk engine chains after it without a copy;
 * `valid` is input 24 (the prefix mask).  Rows of padded (invalid) tokens are written but carry no meaning.
 *
 * Weights, in this order (reference/pi05.py:110-115), all BF16, [out, in] row-major, 16-byte aligned:
 *   0 ln1 [18,2048]   1 ln2 [18,2048]   2 lq [18,2048,2048]   3 lk [18,256,2048]   4 lv [18,256,2048]
 *   5 lo [18,2048,2048]   6 lg [18,16384,2048]   7 lu [18,16384,2048]   8 ld [18,2048,16384]                     */
typedef struct pi05_prefill* pi05_prefill_t;
#define PI05_PREFILL_NUM_WEIGHTS 9
int pi05_prefill_create(int device, int max_tokens, pi05_prefill_t* out);
int pi05_prefill_workspace_bytes(pi05_prefill_t h, size_t* bytes);
/* Records the nine weight pointers (read in place) and the caller-allocated workspace (256-byte aligned). */
int pi05_prefill_bind(pi05_prefill_t h, const void* const weights[PI05_PREFILL_NUM_WEIGHTS], void* workspace,
                      size_t workspace_bytes);
/* One prefill, asynchronous on `stream`: embeddings [tokens, 2048] BF16 (already scaled, as the reference passes them),
 * valid [tokens] bytes (non-zero = valid), keys / values [n_layers.., tokens, 1, 256] BF16 outputs laid out for 18
 * layers ([18, tokens, 1, 256]); n_layers < 18 runs only the first layers (debug). */
int pi05_prefill_run(pi05_prefill_t h, const void* embeddings, const void* valid, int tokens, void* keys, void* values,
                     int n_layers, void* stream);
/* How pi05_prefill_run launches a prefill of `tokens` tokens on a GPU of `sms` SMs, computed on the host (no counterpart
 * in the reference, whose prefill is eager PyTorch; it exists so that these decisions can be tested without a GPU).
 * info = {128-token tiles, 1 when the gate/up, down and O projections run on CTA pairs over 256-token tiles, 1 when the
 * down projection is a stream-K launch, and for that launch its 128 x 256 tiles, k blocks per tile and CTAs (else 0)}.
 * With a stream-K down projection the call also lists the segments {tile, first k block, one past the last} CTA `cta`
 * works through, in order (up to `capacity` triples; *count receives their number): a segment that starts at k block 0
 * makes the CTA the tile's owner, any other one a contributor of partial sums. */
#define PI05_PREFILL_PLAN_INFO 6
int pi05_prefill_plan(int sms, int tokens, int cta, int info[PI05_PREFILL_PLAN_INFO], int* segments, int capacity, int* count);
/* Synchronises `stream` and reports a bounded device-side wait that gave up (PI05_ERR_DEVICE_TIMEOUT), like pi05_status. */
int pi05_prefill_status(pi05_prefill_t h, void* stream, int* code, int* where);
const char* pi05_prefill_last_error(pi05_prefill_t h);
int pi05_prefill_destroy(pi05_prefill_t h);

#ifdef __cplusplus
}
#endif
#endif /* PI05_B200_H_ */

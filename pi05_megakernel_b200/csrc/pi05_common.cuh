// Geometry, shared-memory layout, schedule and parameter types shared by the host code and every variant of the
// chunk kernel.
#pragma once
#include <cuda.h>
#include <cuda_bf16.h>
#include <stdint.h>

namespace pi05 {


// ------------------------------------------------------------------------------------------- geometry
constexpr int T = 50;          // action tokens
constexpr int ADIM = 32;       // action width
constexpr int W = 1024;        // expert width
constexpr int NL = 18;         // expert layers
constexpr int NS = 10;         // Euler steps
constexpr int HD = 256;        // head dim
constexpr int NQH = 8;         // query heads (one KV head)
constexpr int QD = NQH * HD;   // 2048
constexpr int QKVW = QD + 2 * HD;  // 2560: q | k | v
constexpr int FF = 4096;       // MLP width
constexpr int NNORM = 2 * NL + 1;  // adaRMS norms (attn, ffn per layer + final)
constexpr int MODW = 3 * W;        // scale | shift | gate
constexpr float EPS = 1e-6f;

constexpr int THREADS = 256;
constexpr int NROW_CTAS = 25;      // attention / row-op CTAs: two tokens each
constexpr int KATOM = 64;          // K elements per TMA box (128 B of BF16 = one swizzle row)
constexpr int KSTAGE = 128;        // K elements per pipeline stage (two boxes)
constexpr int W_ATOM_BYTES = 128 * 128;  // 128 weight rows x 64 k
constexpr int A_ATOM_BYTES = 64 * 128;   // 64 token rows x 64 k
constexpr int W_STAGE_BYTES = 2 * W_ATOM_BYTES;
constexpr int A_STAGE_BYTES = 2 * A_ATOM_BYTES;
constexpr int A_BOX_ROWS = 50;           // token rows actually copied per activation box
constexpr int A_STAGE_TX = 2 * A_BOX_ROWS * 128;   // bytes a stage's activation half brings in
constexpr int STAGE_BYTES_ALL = W_STAGE_BYTES + A_STAGE_BYTES;   // 48 KB: weights, then activations
constexpr int NSTG = 4;            // pipeline depth (192 KB)
constexpr int STAGE_STRIDE = 72;   // BF16 elements per row of the epilogue exchange buffer (144 B)
constexpr int STAGE_BYTES = 128 * STAGE_STRIDE * 2;

constexpr int OFF_RING = 0;
constexpr int OFF_STAGE = OFF_RING + NSTG * STAGE_BYTES_ALL;   // epilogue exchange buffer; also the prologue's scratch
constexpr int OFF_BARS = OFF_STAGE + STAGE_BYTES;

// shared-memory layout of the row CTAs (attention + row operations).  It may overlap the prologue's scratch
// (OFF_STAGE): the prologue is over before a row CTA touches it.
constexpr int KV_STRIDE = HD + 8;                   // BF16 elements per Q row (528 B: conflict-free ldmatrix)
constexpr int KV_SEG_BYTES = 64 * 128;              // 64 keys x 64 dims, rows of 128 B in the TMA's 128-byte swizzle
constexpr int KV_STAGE_BYTES = 4 * KV_SEG_BYTES;    // one 64-key chunk of K or of V: four such segments
constexpr int ATT_STAGES = 3;                       // 192 keys resident: all of prefix 128 + the 50 suffix keys
constexpr int P_STRIDE = ATT_STAGES * 64 + 8;
constexpr int OFF_KS = 0;
constexpr int OFF_VS = OFF_KS + ATT_STAGES * KV_STAGE_BYTES;
constexpr int OFF_QS = OFF_VS + ATT_STAGES * KV_STAGE_BYTES;
constexpr int OFF_PS = OFF_QS + 16 * KV_STRIDE * 2;
constexpr int OFF_RED = OFF_PS + 16 * P_STRIDE * 2;          // float [8][16]
constexpr int OFF_KVALID = OFF_RED + 8 * 16 * 4;             // uint8 [ATT_STAGES][64]
constexpr int OFF_ATTBARS = OFF_KVALID + ATT_STAGES * 64;   // mbarriers: keys landed [ATT_STAGES], values landed [ATT_STAGES]
static_assert(ATT_STAGES * 64 + 2 * ATT_STAGES * 8 <= 256 && OFF_ATTBARS % 8 == 0, "attention barriers");
constexpr int OFF_ROWBUF = OFF_KVALID + 256;                 // row-op scratch: float [2][1024 + 64]
constexpr int OFF_PAGETAB = OFF_ROWBUF + 2 * (1024 + 64) * 4;   // int [MAX_PAGE_ENTRIES]: the page table of the prefix cache
constexpr int MAX_PAGE_ENTRIES = 1024;                        // batch x pages per observation
constexpr int ATT_SMEM_END = OFF_PAGETAB + MAX_PAGE_ENTRIES * 4;
constexpr int SMEM_BYTES = (ATT_SMEM_END > OFF_BARS + 512 ? ATT_SMEM_END : OFF_BARS + 512) + 1024;   // + alignment slack
static_assert(SMEM_BYTES <= 232448 - 256, "over the 227 KB per-CTA limit");

// stages of one layer pass, in dependency order
enum { ST_QKV = 0, ST_ATT = 1, ST_O = 2, ST_RATT = 3, ST_GU = 4, ST_DOWN = 5, ST_RFFN = 6, NSTAGE = 7 };
enum { G_QKV = 0, G_O = 1, G_GU = 2, G_DOWN = 3 };

// event counters (uint32 each) in the control block
enum { EV_P0 = 0, EV_P1, EV_P2, EV_P3, EV_ANA, EV_QKV, EV_KV, EV_ATT, EV_O, EV_ANF, EV_GU, EV_DOWN, EV_EXIT, EV_PART, EV_PART2, NEVENTS };
// EV_PART / EV_PART2 (key groups, one observation): slot u of the 2 * MAXB slots counts the partial results of row unit u
// every counter sits on its own 128-byte line of the control block; words 0..3 are the status
constexpr int MAXB = 16;            // observations per launch (weights are streamed from HBM once for all of them)
#define EVB(e, b) (32 * (1 + (e) * MAXB + (b)))   // counter of event e for observation b
#define EVW(e) EVB(e, 0)
constexpr int NKVTILES = 4;         // k (2) and v (2) tiles of the QKV GEMM
static_assert(NROW_CTAS <= 2 * MAXB, "EV_PART / EV_PART2 slots");
// Copies of the normalised activations (inputs of the QKV and gate/up GEMMs, read by up to 64 CTAs at the same
// moment): GEMM CTA c reads copy c % AN_COPIES.  Eight copies were measured and changed nothing in the arrival rate
// of the activation stages (the readers are not limited by contention on the same L2 lines), so one copy is kept.
constexpr int AN_COPIES = 1;
constexpr int MAX_KEY_GROUPS = 3;   // row-CTA groups that may share the keys of one attention
constexpr int ATT_PART_FLOATS = 256 * 16 + 16 * 2;   // per (group, unit): every thread's 16 accumulators, then (max, sum) per row
constexpr int CTRL_BYTES = 128 * (1 + NEVENTS * MAXB);

// wait kinds reported in the status word
enum { WAIT_W_EMPTY = 1, WAIT_W_FULL, WAIT_A_EMPTY, WAIT_A_FULL, WAIT_T_EMPTY, WAIT_T_FULL, WAIT_EVENT,
       WAIT_DRAIN };

// gemm: kind in bits 0..6; batched schedules: bit 7 = the entry belongs to the layer pass before the cycle's (two-stream
// schedule), bits 8.. = group of observations + 1 (0: every group in turn)
struct Unit { int gemm, tile, k0, nk; };
constexpr int MAX_UNITS = 32;              // schedule entries per CTA and layer pass
constexpr int MAX_TP = 8;                  // GPUs that may share one chunk (tensor parallel)
// Tensor parallel: every rank holds receive slots [2 reductions (after O, after down)][tp_size ranks][T][W] FP32 and one
// arrival counter per (reduction, row CTA); the peers write into them over NVLink.  Neither is cleared at kernel exit
// (a peer may be a little ahead or behind): the counters only grow, and a launch waits for values above `tp_base`.
constexpr int TP_SLOT_FLOATS = T * W;
constexpr int TP_FLAG_STRIDE = 32;         // one counter per 128-byte line

struct alignas(64) TMaps {
  CUtensorMap wq, wk, wv, wo, wg, wu, wd;   // weights: {K, L*rows} BF16, box {64, 64}, 128-B swizzle
  CUtensorMap an_attn, an_ffn, attn, act;   // activations: {K, 50} BF16 (an_*: AN_COPIES copies per observation), box {64, 50}; slot rows 50..63 are never written
  CUtensorMap pk, pv;                       // prefix keys / values, full pages: {64, page tokens, 4, L, pages} BF16, box {64, 64, 4, 1, 1}
  CUtensorMap pk_tail, pv_tail;             // the same pool, rows limited to the valid tokens of an observation's last page
  CUtensorMap sk, sv;                       // this layer's suffix keys / values: {64, 50, 4, batch}, same box
};

// Pointers that differ from one observation of the batch to the next (b = 0 in Params; obs() advances them).
struct ObsPtrs {
  const float* noise;                       // [T][32]
  const uint8_t* prefix_mask;               // [P]
  float* actions;                           // [T][32]
  float *x, *o_acc, *d_acc;                 // [T][32], [T][W], [T][W]
  float* qkv_acc;                           // [T][2560] split-K accumulator of q (FP32, before rounding and RoPE)
  uint32_t* rope;                           // [T][128]: cos BF16 | sin BF16 << 16
  uint32_t* rope2;                          // [T/2][128][2]: {cos t, cos t+1}, {sin t, sin t+1} BF16 pairs
  __nv_bfloat16 *h, *an_attn, *an_ffn, *k, *v, *attn, *act;   // k, v: [T][256] suffix keys (after RoPE) / values
  int b;
};

struct Params {
  TMaps maps;
  // inputs shared by the whole batch
  const float *ain_w, *ain_b, *tin_w, *tin_b, *tout_w, *tout_b, *aout_w, *aout_b;
  const float *attn_nw, *attn_nb, *ffn_nw, *ffn_nb, *fin_nw, *fin_nb;
  const __nv_bfloat16 *wq, *wk, *wv, *wo, *wg, *wu, *wd;
  ObsPtrs ob;
  // workspace shared by the whole batch
  unsigned int* ctrl;      // [0..3] status, [EVB(e, b)] event counters, one per 128-byte line
  float *temb, *hid, *cond, *mod;
  const Unit* sched;       // [grid][MAX_UNITS]
  const int* sched_n;      // [grid]
  unsigned long long* stamps;
  long long wait_limit;
  int prefix, n_steps, n_layers, max_stage, n_gemm_ctas, batch;
  int row_groups;          // groups of NROW_CTAS row CTAs; group g serves observations g, g + row_groups, ...
  int key_groups;          // one observation, long prefix: the groups split the keys of every attention instead
  const int* page_table;   // [batch][pages_per_obs] physical page of every logical page of the prefix cache
  int pages_per_obs, page_tokens;
  float* att_part;         // [MAX_KEY_GROUPS - 1][NROW_CTAS][ATT_PART_FLOATS] partial attention results of groups >= 1
  int poll_ns;             // pause between two samples of a stage counter
  int drop_event;          // debug: this event is never signalled (exercises the bounded waits); -1 = none
  int stream_split;        // two-stream schedule: groups below this index form stream A, the rest stream B (0: one stream)
  int row_order;           // several observations: 0 = attention of one, then the residual of the one before; 1 = all attentions first
  int cta_perm;            // role permutation over the blocks of the grid (see the kernel's first lines)
  int n_units[4];          // units per GEMM kind (event targets)
  // tensor parallel (tp_size > 1): this rank's receive slots and arrival counters, and where every peer's are
  int tp_rank, tp_size;
  unsigned int tp_base;    // arrivals per counter that earlier launches of this binding have consumed
  float* tp_recv;          // [2][tp_size][T][W]
  unsigned int* tp_flags;  // [2][NROW_CTAS] counters, TP_FLAG_STRIDE words apart
  float* tp_peer_recv[MAX_TP];
  unsigned int* tp_peer_flags[MAX_TP];
  float t_steps[NS];
  float dt;
};

}  // namespace pi05
